"""Thin Python handle over the C-ABI device planner (``rt_plan_*``).

All planning happens in the CUDA kernels behind the C ABI; this class only
owns the handle and turns numpy / torch buffers into pointers.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .workloads import Layout


def _is_i32(x) -> bool:
    """True for int32 ids, False for int64; anything else is refused."""
    name = str(x.dtype)
    if name in ("int32", "torch.int32"):
        return True
    if name in ("int64", "torch.int64"):
        return False
    raise TypeError(f"slot ids must be int32 or int64, not {name}")


def _ptr(x):
    """Raw address of a torch tensor, numpy array or None."""
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    return C.c_void_p(x.ctypes.data)


class DevicePlanner:
    def __init__(self, layout: Layout, device: int = 0, *, max_indices: int = 0,
                 max_ranges: int = 1 << 16):
        self.layout = layout
        self.device = device
        self.max_ranges = max_ranges
        bg = np.ascontiguousarray(layout.buffer_group(), dtype=np.uint32)
        self._bg = bg
        lay = capi.Layout(layout.n_buffers, layout.n_groups, layout.alloc_bytes,
                          layout.bytes_per_slot, layout.block_bytes, layout.capacity,
                          bg.ctypes.data_as(C.POINTER(C.c_uint32)) if layout.n_groups > 1 else None,
                          device, 0)
        handle = C.c_void_p()
        capi.check(capi.lib.rt_plan_create(C.byref(lay), device, max_indices, max_ranges,
                                           C.byref(handle)), "rt_plan_create")
        self._h = handle

    def close(self):
        if getattr(self, "_h", None):
            lib = getattr(capi, "lib", None)     # gone when the interpreter is shutting down
            if lib is not None:
                lib.rt_plan_destroy(self._h)
            self._h = None

    __del__ = close

    # ---- resident bitmaps -------------------------------------------------
    def set_resident(self, block_sets):
        words = np.zeros((self.layout.n_groups, capi.RT_BITMAP_WORDS), dtype=np.uint32)
        for g, blocks in enumerate(block_sets):
            for b in blocks:
                words[g, b >> 5] |= np.uint32(1 << (b & 31))
        capi.check(capi.lib.rt_plan_set_resident(self._h, _ptr(words)), "rt_plan_set_resident")

    def get_resident(self):
        words = np.zeros((self.layout.n_groups, capi.RT_BITMAP_WORDS), dtype=np.uint32)
        capi.check(capi.lib.rt_plan_get_resident(self._h, _ptr(words)), "rt_plan_get_resident")
        return [bitmap_to_blocks(w) for w in words]

    # ---- planning ---------------------------------------------------------
    def step_host(self, slots: np.ndarray, group_off: np.ndarray, budget: int, flags: int = 0,
                  *, out: np.ndarray | None = None, raise_on_slot_range: bool = True):
        """Host buffers in, host ranges out (copies inside). Returns (ranges, result)."""
        assert group_off.dtype == np.int64
        if out is None:
            out = np.empty(self.max_ranges, dtype=capi.RANGE_DTYPE)
        res = capi.PlanResult()
        fn = capi.lib.rt_plan_step_i32 if _is_i32(slots) else capi.lib.rt_plan_step
        st = fn(self._h, _ptr(slots), _ptr(group_off), budget, flags,
                                   _ptr(out), len(out), C.byref(res))
        if st == capi.RT_ERR_SLOT_RANGE and not raise_on_slot_range:
            st = 0
        capi.check(st, "rt_plan_step")
        return out[:min(res.n_ranges, len(out))], res

    def narrow_threads(self) -> int:
        """Host threads `step_host` narrows 64-bit ids with (0: it copies them as they are)."""
        t = C.c_uint32()
        capi.check(capi.lib.rt_plan_narrow_threads(self._h, C.byref(t)), "rt_plan_narrow_threads")
        return t.value

    def step_device(self, d_slots, group_off: np.ndarray, budget: int, flags: int, d_out, d_result,
                    stream=None):
        """Everything already on the device (torch tensors); asynchronous.
        ``d_slots`` may be int64 or int32."""
        cap = d_out.numel() * d_out.element_size() // capi.RANGE_DTYPE.itemsize
        fn = capi.lib.rt_plan_step_device_i32 if _is_i32(d_slots) else capi.lib.rt_plan_step_device
        capi.check(fn(
            self._h, _ptr(d_slots), _ptr(group_off), budget, flags, _ptr(d_out), cap,
            _ptr(d_result), C.c_void_p(stream) if stream else None), "rt_plan_step_device")

    def step_table(self, d_table, d_lens, budget: int, flags: int, d_out, d_result, stream=None):
        rows, stride = d_table.shape
        cap = d_out.numel() * d_out.element_size() // capi.RANGE_DTYPE.itemsize
        fn = capi.lib.rt_plan_step_table_i32 if _is_i32(d_table) else capi.lib.rt_plan_step_table
        capi.check(fn(
            self._h, _ptr(d_table), _ptr(d_lens), rows, stride, budget, flags, _ptr(d_out), cap,
            _ptr(d_result), C.c_void_p(stream) if stream else None), "rt_plan_step_table")

    def scan(self, d_slots, group_off: np.ndarray, d_bitmaps, d_result, stream=None):
        fn = capi.lib.rt_scan_slots_i32 if _is_i32(d_slots) else capi.lib.rt_scan_slots
        capi.check(fn(
            self._h, _ptr(d_slots), _ptr(group_off), _ptr(d_bitmaps), _ptr(d_result),
            C.c_void_p(stream) if stream else None), "rt_scan_slots")

    def from_bitmaps(self, d_want, budget: int, flags: int, d_out, d_result, stream=None):
        cap = d_out.numel() * d_out.element_size() // capi.RANGE_DTYPE.itemsize
        capi.check(capi.lib.rt_plan_from_bitmaps(
            self._h, _ptr(d_want), budget, flags, _ptr(d_out), cap, _ptr(d_result),
            C.c_void_p(stream) if stream else None), "rt_plan_from_bitmaps")

    def sync(self):
        capi.check(capi.lib.rt_plan_sync(self._h), "rt_plan_sync")


def bitmap_to_blocks(words) -> list[int]:
    out = []
    for w, v in enumerate(np.asarray(words, dtype=np.uint32)):
        v = int(v)
        while v:
            b = (v & -v).bit_length() - 1
            out.append(w * 32 + b)
            v &= v - 1
    return out


def blocks_to_bitmap(blocks) -> np.ndarray:
    words = np.zeros(capi.RT_BITMAP_WORDS, dtype=np.uint32)
    for b in blocks:
        words[b >> 5] |= np.uint32(1 << (b & 31))
    return words


def ranges_to_tuples(ranges: np.ndarray):
    return [(int(r["buffer"]), int(r["dst"]), int(r["offset"]), int(r["bytes"])) for r in ranges]


def result_from_tensor(t) -> dict:
    """Decode an rt_plan_result held in a 64-byte torch uint8 tensor."""
    raw = bytes(t.cpu().numpy().tobytes())
    return capi.PlanResult.from_buffer_copy(raw).as_dict()


def ranges_from_tensor(t, n: int) -> np.ndarray:
    raw = t.cpu().numpy().view(np.uint8).reshape(-1)[:n * capi.RANGE_DTYPE.itemsize]
    return np.frombuffer(raw.tobytes(), dtype=capi.RANGE_DTYPE)
