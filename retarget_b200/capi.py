"""ctypes binding of ``include/retarget_b200.h``.

The shared library is the product; this file only declares its signatures.
If the library has not been built, importing this module raises: there is no
Python or CPU stand-in for the CUDA path.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

import os

PKG = Path(__file__).resolve().parent
# RETARGET_B200_LIB selects another build of the same library (e.g. an experimental variant)
LIB_PATH = Path(os.environ.get("RETARGET_B200_LIB") or PKG / "libretarget_b200.so")

RT_MAX_GROUPS = 128
RT_MAX_BLOCKS = 1024
RT_MAX_BUFFERS = 1024
RT_BITMAP_WORDS = 32
RT_DST_CPU = -1
RT_INITIAL = (1 << 64) - 1

RT_PLAN_EVICT = 1
RT_PLAN_DRY_RUN = 2
RT_PLAN_TMA = 4
RT_PLAN_CHAINED = 8
RT_PLAN_WIDE_COPY = 16

RT_RESULT_OVERFLOW = 1
RT_RESULT_SLOT_RANGE = 2
RT_RESULT_TIMEOUT = 4

RT_OK = 0
RT_ERR_INVALID_ARGUMENT = -1
RT_ERR_NO_DEVICE = -2
RT_ERR_CAPACITY = -5
RT_ERR_ALIGNMENT = -6
RT_ERR_SLOT_RANGE = -7
RT_ERR_IO = -10
RT_ERR_PLAN = -11
RT_ERR_TIMEOUT = -12
RT_ERR_SPEC_POSITIVE = -20
RT_ERR_COMPLETED_COUNT = -27
RT_ERR_BUDGET_DIVISIBLE = -28
RT_ERR_BLOCK_PAGE = -29
RT_ERR_METRICS_MISSING = -30
RT_ERR_METRICS_INVALID = -31
RT_ERR_METRICS_KEY_RUNNING = -32
RT_ERR_METRICS_KEY_QUEUE = -33
RT_ERR_LAYOUT_MISMATCH = -34
RT_ERR_SLOT_SPEC = -35
RT_ERR_FEEDBACK_IDENTITY = -36

UPDATE_MODES = ("incremental", "initial_only", "full_cache")


class UvmConfig(C.Structure):
    """rt_uvm_config: how the in-process UVM server and its prefetch executor run."""
    _fields_ = [("socket_path", C.c_char_p), ("chunk_bytes", C.c_uint64), ("batch_bytes", C.c_uint64),
                ("streams", C.c_uint32), ("listen", C.c_int32), ("overlap_phases", C.c_uint32),
                ("reserved", C.c_uint32)]


class RtError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class WindowSpecStruct(C.Structure):
    _fields_ = [("allocation_bytes", C.c_uint64), ("allocation_count", C.c_uint64),
                ("bytes_per_token", C.c_uint64), ("width_tokens", C.c_uint64),
                ("lookahead_tokens", C.c_uint64), ("quantum_tokens", C.c_uint64),
                ("min_update_seconds", C.c_double), ("idle_only", C.c_int32),
                ("update_mode", C.c_int32)]


class AllocInfo(C.Structure):
    _fields_ = [("id", C.c_uint64), ("bytes", C.c_uint64), ("device", C.c_int32),
                ("concurrent", C.c_int32)]


class Metrics(C.Structure):
    _fields_ = [("prompt_tokens_total", C.c_double), ("generation_tokens_total", C.c_double),
                ("num_running_reqs", C.c_double), ("num_queue_reqs", C.c_double),
                ("present", C.c_uint32), ("reserved", C.c_uint32)]


class WindowUpdate(C.Structure):
    _fields_ = [("full", C.c_int32), ("refresh", C.c_int32), ("old_window", C.c_uint64 * 2),
                ("new_window", C.c_uint64 * 2), ("generation", C.c_uint64), ("cache_count", C.c_uint64),
                ("gpu_bytes", C.c_uint64), ("cpu_bytes", C.c_uint64), ("completed_highwater", C.c_double)]


class WindowState(C.Structure):
    _fields_ = [("has_current", C.c_int32), ("has_signature", C.c_int32), ("current", C.c_uint64 * 2),
                ("last_update", C.c_double), ("completed_highwater", C.c_double),
                ("signature_count", C.c_uint64)]


class SlotSpecStruct(C.Structure):
    _fields_ = [("block_tokens", C.c_uint64), ("lookahead_tokens", C.c_uint64),
                ("min_update_seconds", C.c_double), ("max_blocks_per_update", C.c_uint64),
                ("active_seconds", C.c_double), ("refresh_seconds", C.c_double),
                ("max_feedback_lag_seconds", C.c_double)]


class BlockStamp(C.Structure):
    _fields_ = [("block", C.c_uint32), ("reserved", C.c_uint32), ("t", C.c_double)]


class SnapshotDoc(C.Structure):
    _fields_ = [("pid", C.c_uint64), ("epoch", C.c_uint64), ("block_tokens", C.c_uint64),
                ("sequence", C.c_int64), ("observed_monotonic_s", C.c_double),
                ("published_monotonic_s", C.c_double),
                ("block_versions", C.POINTER(C.c_int32)), ("n_versions", C.c_size_t),
                ("recent_reads", C.POINTER(BlockStamp)), ("n_reads", C.c_size_t),
                ("recent_writes", C.POINTER(BlockStamp)), ("n_writes", C.c_size_t),
                ("free_head_blocks", C.POINTER(C.c_uint32)), ("n_free", C.c_size_t)]


class SlotUpdate(C.Structure):
    _fields_ = [("generation", C.c_uint64), ("epoch", C.c_uint64), ("sequence", C.c_int64),
                ("observed_monotonic_s", C.c_double), ("cache_count", C.c_uint64), ("gpu_bytes", C.c_uint64),
                ("n_desired", C.c_uint64), ("n_selected", C.c_uint64)]


class SlotState(C.Structure):
    _fields_ = [("has_epoch", C.c_int32), ("reserved", C.c_int32), ("epoch", C.c_uint64),
                ("last_attempt", C.c_double), ("committed_count", C.c_uint64)]


class BlockCommit(C.Structure):
    _fields_ = [("block", C.c_uint32), ("version", C.c_int32), ("at", C.c_double)]


class IdRange(C.Structure):
    _fields_ = [("id", C.c_uint64), ("offset", C.c_uint64), ("bytes", C.c_uint64),
                ("dst", C.c_int32), ("reserved", C.c_int32)]


class Range(C.Structure):
    _fields_ = [("buffer", C.c_uint32), ("dst", C.c_int32), ("offset", C.c_uint64),
                ("bytes", C.c_uint64)]


RANGE_DTYPE = np.dtype([("buffer", "<u4"), ("dst", "<i4"), ("offset", "<u8"), ("bytes", "<u8")])
assert RANGE_DTYPE.itemsize == C.sizeof(Range) == 24


class Layout(C.Structure):
    _fields_ = [("n_buffers", C.c_uint32), ("n_groups", C.c_uint32), ("alloc_bytes", C.c_uint64),
                ("bytes_per_slot", C.c_uint32), ("block_bytes", C.c_uint32),
                ("capacity_slots", C.c_uint64), ("buffer_group", C.POINTER(C.c_uint32)),
                ("dst_device", C.c_int32), ("reserved", C.c_int32)]


class PlanResult(C.Structure):
    _fields_ = [("n_ranges", C.c_uint32), ("n_cpu_ranges", C.c_uint32), ("flags", C.c_uint32),
                ("blocks_touched", C.c_uint32), ("blocks_desired", C.c_uint32),
                ("blocks_added", C.c_uint32), ("blocks_evicted", C.c_uint32),
                ("reserved", C.c_uint32), ("invalid_slots", C.c_uint64),
                ("ignored_slots", C.c_uint64), ("gpu_bytes", C.c_uint64), ("cpu_bytes", C.c_uint64)]

    def as_dict(self):
        return {k: int(getattr(self, k)) for k, _ in self._fields_ if k != "reserved"}


assert C.sizeof(PlanResult) == 64


def _load():
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m retarget_b200.build` "
            "(needs nvcc). retarget_b200 has no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    u64p, u32p, i64p = C.POINTER(C.c_uint64), C.POINTER(C.c_uint32), C.POINTER(C.c_int64)
    sig = {
        "rt_strerror": (C.c_char_p, [C.c_int]),
        "rt_abi_version": (C.c_int, []),
        "rt_last_cuda_error": (C.c_int, []),
        "rt_window_spec_check": (C.c_int, [C.POINTER(WindowSpecStruct), C.POINTER(C.c_int)]),
        "rt_window": (C.c_int, [C.POINTER(WindowSpecStruct), C.c_double, u64p]),
        "rt_interval_difference": (C.c_int, [u64p, u64p, u64p]),
        "rt_aligned_target": (C.c_int, [C.POINTER(C.c_uint64), C.c_size_t, C.c_uint64, C.c_uint64,
                                        C.POINTER(C.c_uint64)]),
        "rt_window_accounting": (C.c_int, [C.POINTER(WindowSpecStruct), C.c_uint64, C.c_uint64,
                                           u64p, u64p, C.c_int, C.c_int, u64p, u64p]),
        "rt_slot_budget": (C.c_int, [C.POINTER(WindowSpecStruct), C.c_uint64, u64p]),
        "rt_encode_mask": (C.c_int, [u32p, C.c_size_t, C.c_char_p, C.c_size_t]),
        "rt_encode_runs": (C.c_int, [i64p, C.c_size_t, i64p, C.c_size_t, C.POINTER(C.c_size_t)]),
        "rt_expand_command": (C.c_int, [C.POINTER(AllocInfo), C.c_size_t, C.c_uint64, C.c_char_p,
                                        C.c_uint64, C.POINTER(IdRange), C.c_size_t,
                                        C.POINTER(C.c_size_t), C.POINTER(C.c_char_p)]),
        "rt_plan_create": (C.c_int, [C.POINTER(Layout), C.c_int, C.c_uint64, C.c_uint32,
                                     C.POINTER(C.c_void_p)]),
        "rt_plan_destroy": (C.c_int, [C.c_void_p]),
        "rt_plan_set_resident": (C.c_int, [C.c_void_p, C.c_void_p]),
        "rt_plan_get_resident": (C.c_int, [C.c_void_p, C.c_void_p]),
        "rt_plan_step_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                          C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]),
        "rt_plan_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                   C.c_void_p, C.c_uint32, C.c_void_p]),
        "rt_plan_step_table": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64,
                                         C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p,
                                         C.c_void_p]),
        "rt_scan_slots": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p]),
        "rt_plan_step_device_i32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                              C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]),
        "rt_plan_step_i32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                       C.c_void_p, C.c_uint32, C.c_void_p]),
        "rt_plan_step_table_i32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64,
                                             C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p,
                                             C.c_void_p]),
        "rt_scan_slots_i32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_void_p]),
        "rt_plan_from_bitmaps": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p,
                                           C.c_uint32, C.c_void_p, C.c_void_p]),
        "rt_plan_sync": (C.c_int, [C.c_void_p]),
        # controllers
        "rt_window_controller_create": (C.c_int, [C.POINTER(WindowSpecStruct), C.POINTER(C.c_void_p)]),
        "rt_window_controller_destroy": (C.c_int, [C.c_void_p]),
        "rt_window_controller_due": (C.c_int, [C.c_void_p, C.POINTER(Metrics), C.c_double]),
        "rt_window_controller_begin": (C.c_int, [C.c_void_p, C.POINTER(Metrics), C.c_double, C.c_int]),
        "rt_window_controller_plan": (C.c_int, [C.c_void_p, C.POINTER(AllocInfo), C.c_size_t, C.c_uint64,
                                                C.c_char_p, C.c_size_t, C.POINTER(WindowUpdate)]),
        "rt_window_controller_commit": (C.c_int, [C.c_void_p, C.c_double]),
        "rt_window_controller_fail": (C.c_int, [C.c_void_p]),
        "rt_window_controller_get": (C.c_int, [C.c_void_p, C.POINTER(WindowState)]),
        "rt_window_controller_set": (C.c_int, [C.c_void_p, C.POINTER(WindowState)]),
        "rt_window_controller_get_signature": (C.c_int, [C.c_void_p, C.POINTER(AllocInfo), C.c_size_t,
                                                         C.POINTER(C.c_size_t)]),
        "rt_window_controller_set_signature": (C.c_int, [C.c_void_p, C.POINTER(AllocInfo), C.c_size_t, C.c_int]),
        "rt_slot_spec_check": (C.c_int, [C.POINTER(SlotSpecStruct), C.POINTER(C.c_int)]),
        "rt_target_blocks": (C.c_int, [C.POINTER(SnapshotDoc), C.POINTER(SlotSpecStruct), C.c_uint64, C.c_double,
                                       u32p, C.c_size_t, C.POINTER(C.c_size_t)]),
        "rt_slot_controller_create": (C.c_int, [C.POINTER(WindowSpecStruct), C.POINTER(SlotSpecStruct), C.c_uint64,
                                                C.POINTER(C.c_void_p)]),
        "rt_slot_controller_destroy": (C.c_int, [C.c_void_p]),
        "rt_slot_controller_window": (C.c_void_p, [C.c_void_p]),
        "rt_slot_controller_budget": (C.c_uint64, [C.c_void_p]),
        "rt_slot_controller_accept": (C.c_int, [C.c_void_p, C.POINTER(SnapshotDoc)]),
        "rt_slot_controller_choose": (C.c_int, [C.c_void_p, C.POINTER(SnapshotDoc), C.c_double, u32p, C.c_size_t,
                                                C.POINTER(C.c_size_t), u32p, C.c_size_t, C.POINTER(C.c_size_t)]),
        "rt_slot_controller_due": (C.c_int, [C.c_void_p, C.POINTER(SnapshotDoc), C.c_double]),
        "rt_slot_controller_attempt_allowed": (C.c_int, [C.c_void_p, C.c_double]),
        "rt_slot_controller_begin": (C.c_int, [C.c_void_p, C.POINTER(SnapshotDoc), C.c_double]),
        "rt_slot_controller_plan": (C.c_int, [C.c_void_p, C.POINTER(AllocInfo), C.c_size_t, C.c_uint64,
                                              C.c_char_p, C.c_size_t, C.POINTER(SlotUpdate)]),
        "rt_slot_controller_pending": (C.c_int, [C.c_void_p, u32p, C.c_size_t, u32p, C.c_size_t]),
        "rt_slot_controller_commit": (C.c_int, [C.c_void_p, C.c_double]),
        "rt_slot_controller_fail": (C.c_int, [C.c_void_p]),
        "rt_slot_controller_seed": (C.c_int, [C.c_void_p, C.POINTER(SnapshotDoc), C.c_double]),
        "rt_slot_controller_get": (C.c_int, [C.c_void_p, C.POINTER(SlotState)]),
        "rt_slot_controller_set": (C.c_int, [C.c_void_p, C.POINTER(SlotState)]),
        "rt_slot_controller_get_committed": (C.c_int, [C.c_void_p, C.POINTER(BlockCommit), C.c_size_t,
                                                       C.POINTER(C.c_size_t)]),
        "rt_slot_controller_set_committed": (C.c_int, [C.c_void_p, C.POINTER(BlockCommit), C.c_size_t]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def strerror(status: int) -> str:
    return lib.rt_strerror(status).decode()


def check(status: int, what: str = "") -> int:
    if status < 0:
        raise RtError(status, f"{what + ': ' if what else ''}{strerror(status)} (status {status}, "
                              f"cuda {lib.rt_last_cuda_error()})")
    return status


def window_spec_struct(allocation_bytes, allocation_count, bytes_per_token, width_tokens,
                       lookahead_tokens, quantum_tokens, min_update_seconds=1.0, idle_only=True,
                       update_mode="incremental") -> WindowSpecStruct:
    return WindowSpecStruct(allocation_bytes, allocation_count, bytes_per_token, width_tokens,
                            lookahead_tokens, quantum_tokens, float(min_update_seconds),
                            int(bool(idle_only)), UPDATE_MODES.index(update_mode))


def expand_command(registry, generation: int, line: str, page: int = 4096):
    """Returns ``(ranges, None)`` or ``(None, error_string)``; ranges are
    ``(id, offset, bytes, dst)`` tuples in queue order."""
    arr = (AllocInfo * max(1, len(registry)))()
    for k, a in enumerate(registry):
        arr[k] = AllocInfo(a["id"], a["bytes"], a["device"], int(a.get("concurrent", 1)))
    cap = 4096
    while True:
        out = (IdRange * cap)()
        n = C.c_size_t(0)
        err = C.c_char_p()
        st = lib.rt_expand_command(arr, len(registry), generation, line.encode("ascii"), page,
                                   out, cap, C.byref(n), C.byref(err))
        if st == RT_ERR_PLAN:
            return None, err.value.decode()
        if st == RT_ERR_CAPACITY:
            cap = n.value
            continue
        check(st, "rt_expand_command")
        return [(r.id, r.offset, r.bytes, r.dst) for r in out[:n.value]], None
