"""Slot-feedback block placement: the scheduler-facing controller.

Drop-in for the reference's experiments/slot_placement.py: ``SlotPlacementSpec``,
``target_blocks``, ``encode_mask`` and ``SlotPlacementController`` keep their
names, arguments, error behaviour, socket commands and result dictionaries.
Ranking, selection, the record of what was sent, the command line and the
accounting are the native library's (``rt_target_blocks``, ``rt_encode_mask``,
``rt_slot_controller_*``); this file binds them: it reads the snapshot document,
hands it over as arrays, sends the command the library wrote and turns status
codes back into the reference's exceptions.

The controller consumes feedback snapshots (the JSON documents described in
experiments/slot_feedback.py:86-91).  They can come from the reference's file
drop (``RETARGET_SLOT_FEEDBACK_DIR/<pid>.json``) or from any callable passed as
``snapshot_source`` -- e.g. ``DeviceFeedback.snapshot`` of this package, which
keeps the same state in GPU memory and needs no file hop.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import json
import math
import os
import time
from pathlib import Path

from . import capi
from .cache_window import CacheWindowController, _raise_policy, _registry_array
from .control import ControlError


_SPEC_FIELDS = ("block_tokens", "lookahead_tokens", "min_update_seconds", "max_blocks_per_update",
                "active_seconds", "refresh_seconds", "max_feedback_lag_seconds")


@dataclasses.dataclass(frozen=True)
class SlotPlacementSpec:
    """experiments/slot_placement.py:18-34"""
    block_tokens: int = 256
    lookahead_tokens: int = 4096
    min_update_seconds: float = .25
    max_blocks_per_update: int = 4
    active_seconds: float = 2.0
    refresh_seconds: float = 10.0
    max_feedback_lag_seconds: float = 1.0

    def __post_init__(self):
        # what depends on Python types is checked here, the ranges by the library;
        # the reference checks the three integers first, then the four intervals
        ints = ("block_tokens", "lookahead_tokens", "max_blocks_per_update")
        for key in ints:
            value = getattr(self, key)
            if type(value) is not int or value <= 0 or value >= 1 << 63:
                raise ValueError(key)
        raw = capi.SlotSpecStruct(*(float(getattr(self, k)) if k not in ints else getattr(self, k)
                                    for k in _SPEC_FIELDS))
        bad = C.c_int(-1)
        if capi.lib.rt_slot_spec_check(C.byref(raw), C.byref(bad)):
            raise ValueError(_SPEC_FIELDS[bad.value])
        object.__setattr__(self, "_raw", raw)

    def _struct(self) -> capi.SlotSpecStruct:
        return self._raw


class _SnapshotArrays:
    """A snapshot document as the arrays of rt_snapshot_doc (kept alive with it)."""

    def __init__(self, data):
        versions = data["block_versions"]
        reads, writes, free = data["recent_reads"], data["recent_writes"], data["free_head_blocks"]
        self.versions = (C.c_int32 * max(1, len(versions)))(*versions)
        self.reads = (capi.BlockStamp * max(1, len(reads)))(*[capi.BlockStamp(int(b), 0, float(t)) for b, t in reads])
        self.writes = (capi.BlockStamp * max(1, len(writes)))(*[capi.BlockStamp(int(b), 0, float(t)) for b, t in writes])
        self.free = (C.c_uint32 * max(1, len(free)))(*free)
        self.doc = capi.SnapshotDoc(
            int(data.get("pid", 0)), int(data.get("epoch", 0)), int(data.get("block_tokens", 0)),
            int(data.get("sequence", 0)), float(data.get("observed_monotonic_s", 0.0)),
            float(data.get("published_monotonic_s", 0.0)),
            self.versions, len(versions), self.reads, len(reads), self.writes, len(writes), self.free, len(free))

    def ref(self):
        return C.byref(self.doc)


def target_blocks(snapshot, spec, budget, now):
    """experiments/slot_placement.py:37-44"""
    arrays = _SnapshotArrays(snapshot)
    cap = len(snapshot["recent_reads"]) + len(snapshot["recent_writes"]) + len(snapshot["free_head_blocks"]) + 1
    out = (C.c_uint32 * cap)()
    n = C.c_size_t()
    capi.check(capi.lib.rt_target_blocks(arrays.ref(), C.byref(spec._struct()), int(budget), float(now),
                                         out, cap, C.byref(n)), "rt_target_blocks")
    return [int(b) for b in out[:n.value]]


def encode_mask(blocks) -> str:
    """experiments/slot_placement.py:47-51"""
    blocks = list(blocks)
    arr = (C.c_uint32 * max(1, len(blocks)))(*blocks)
    cap = (max(blocks) // 4 + 3) if blocks else 3
    buf = C.create_string_buffer(cap)
    capi.check(capi.lib.rt_encode_mask(arr, len(blocks), buf, cap), "rt_encode_mask")
    return buf.value.decode()


class SlotPlacementController(CacheWindowController):
    """experiments/slot_placement.py:55-162.  ``committed``, ``epoch`` and
    ``last_attempt`` are held by the native controller and shown as attributes.

    ``snapshot_source``: a callable ``now -> snapshot document or None`` used
    instead of the file drop (``RETARGET_SLOT_FEEDBACK_DIR/<pid>.json``)."""

    def __init__(self, cache_spec, slot_spec, pid, snapshot_source=None):
        self.spec = cache_spec
        self.slot_spec = slot_spec
        self.pid = pid
        self._source = snapshot_source
        if snapshot_source is None:
            self.feedback_path = Path(os.environ["RETARGET_SLOT_FEEDBACK_DIR"]) / f"{pid}.json"
        handle = C.c_void_p()
        status = capi.lib.rt_slot_controller_create(C.byref(cache_spec._struct()), C.byref(slot_spec._struct()),
                                                    int(pid), C.byref(handle))
        if status in (capi.RT_ERR_BUDGET_DIVISIBLE, capi.RT_ERR_BLOCK_PAGE):
            raise ValueError(capi.strerror(status))
        capi.check(status, "rt_slot_controller_create")
        self._s = handle
        # the window controller this one extends lives inside the native object
        self._owner = False
        self._w = C.c_void_p(capi.lib.rt_slot_controller_window(self._s))
        self.budget = int(capi.lib.rt_slot_controller_budget(self._s))

    def __del__(self):
        lib = getattr(capi, "lib", None)
        if getattr(self, "_s", None) and lib is not None:
            lib.rt_slot_controller_destroy(self._s)
            self._s = None

    # ---- state ----
    def _slot_state(self) -> capi.SlotState:
        st = capi.SlotState()
        capi.check(capi.lib.rt_slot_controller_get(self._s, C.byref(st)))
        return st

    @property
    def committed(self):
        cap = max(1, int(self._slot_state().committed_count))
        arr = (capi.BlockCommit * cap)()
        n = C.c_size_t()
        capi.check(capi.lib.rt_slot_controller_get_committed(self._s, arr, cap, C.byref(n)))
        return {int(e.block): (int(e.version), float(e.at)) for e in arr[:n.value]}

    @committed.setter
    def committed(self, record):
        items = list(record.items())
        arr = (capi.BlockCommit * max(1, len(items)))(*[capi.BlockCommit(int(b), int(v), float(t))
                                                       for b, (v, t) in items])
        capi.check(capi.lib.rt_slot_controller_set_committed(self._s, arr, len(items)))

    @property
    def epoch(self):
        st = self._slot_state()
        return int(st.epoch) if st.has_epoch else None

    @epoch.setter
    def epoch(self, value):
        st = self._slot_state()
        st.has_epoch, st.epoch = int(value is not None), int(value or 0)
        capi.check(capi.lib.rt_slot_controller_set(self._s, C.byref(st)))

    @property
    def last_attempt(self):
        return float(self._slot_state().last_attempt)

    @last_attempt.setter
    def last_attempt(self, t):
        st = self._slot_state()
        st.last_attempt = float(t)
        capi.check(capi.lib.rt_slot_controller_set(self._s, C.byref(st)))

    # ---- policy ----
    def snapshot(self, now):
        """The current snapshot document, or None when there is none to act on
        (no file yet, or published too long after it was observed)."""
        if self._source is not None:
            data = self._source(now)
            if data is None:
                return None
        else:
            try:
                data = json.loads(self.feedback_path.read_text())
            except FileNotFoundError:
                return None
        verdict = capi.lib.rt_slot_controller_accept(self._s, _SnapshotArrays(data).ref())
        if verdict == capi.RT_ERR_FEEDBACK_IDENTITY:
            raise ControlError(capi.strerror(verdict))
        capi.check(verdict, "rt_slot_controller_accept")
        return data if verdict else None

    def choose(self, snapshot, now):
        arrays = _SnapshotArrays(snapshot)
        cap = max(1, self.budget)
        desired, selected = (C.c_uint32 * cap)(), (C.c_uint32 * cap)()
        nd, ns = C.c_size_t(), C.c_size_t()
        status = capi.lib.rt_slot_controller_choose(self._s, arrays.ref(), float(now), desired, cap, C.byref(nd),
                                                    selected, cap, C.byref(ns))
        if status == capi.RT_ERR_INVALID_ARGUMENT:
            raise IndexError("snapshot has no version for a desired block")
        capi.check(status, "rt_slot_controller_choose")
        return [int(b) for b in desired[:nd.value]], [int(b) for b in selected[:ns.value]]

    def due(self, metrics, now):
        if not capi.check(capi.lib.rt_slot_controller_attempt_allowed(self._s, float(now))):
            return False
        snapshot = self.snapshot(now)
        arrays = None if snapshot is None else _SnapshotArrays(snapshot)
        status = capi.lib.rt_slot_controller_due(self._s, arrays.ref() if arrays else None, float(now))
        return bool(capi.check(status, "rt_slot_controller_due"))

    def update(self, uvm, metrics, now, *, initial=False):
        lib = capi.lib
        if initial:
            result = super().update(uvm, metrics, now, initial=True)
            snapshot = self.snapshot(time.monotonic())
            if snapshot is None:
                raise ControlError("slot feedback unavailable after model warmup")
            capi.check(lib.rt_slot_controller_seed(self._s, _SnapshotArrays(snapshot).ref(), time.monotonic()),
                       "rt_slot_controller_seed")
            result.update(placement_kind="slot_feedback", committed_blocks=sorted(self.committed),
                          block_tokens=self.slot_spec.block_tokens, feedback_epoch=self.epoch)
            return result
        # the attempt is stamped before the snapshot is looked at, as in the reference
        self.last_attempt = now
        snapshot = self.snapshot(now)
        arrays = None if snapshot is None else _SnapshotArrays(snapshot)
        go = capi.check(lib.rt_slot_controller_begin(self._s, arrays.ref() if arrays else None, float(now)),
                        "rt_slot_controller_begin")
        if not go:
            return None
        generation, allocations = uvm._allocation_snapshot()
        command = C.create_string_buffer(512)
        plan = capi.SlotUpdate()
        status = lib.rt_slot_controller_plan(self._s, _registry_array(allocations), len(allocations),
                                             int(generation), command, len(command), C.byref(plan))
        if status == capi.RT_ERR_LAYOUT_MISMATCH:
            raise ControlError("slot-placement cache geometry changed")
        capi.check(status, "rt_slot_controller_plan")
        desired, selected = (C.c_uint32 * max(1, plan.n_desired))(), (C.c_uint32 * max(1, plan.n_selected))()
        capi.check(lib.rt_slot_controller_pending(self._s, desired, plan.n_desired, selected, plan.n_selected))
        desired, selected = [int(b) for b in desired[:plan.n_desired]], [int(b) for b in selected[:plan.n_selected]]
        uvm.wait_idle(timeout=600)
        reply = uvm.command(command.value.decode("ascii"))
        if not reply.get("ok"):
            lib.rt_slot_controller_fail(self._s)
            raise ControlError(f"slot prefetch rejected: {reply}")
        try:
            status = uvm._wait_job(int(reply["job_id"]), timeout=600)
        except Exception:
            lib.rt_slot_controller_fail(self._s)
            raise
        commit = time.monotonic()
        capi.check(lib.rt_slot_controller_commit(self._s, commit), "rt_slot_controller_commit")
        return dict(initial=False, placement_kind="slot_feedback", update_mode="slot_feedback",
                    allocation_generation=generation, feedback_epoch=int(plan.epoch),
                    feedback_sequence=snapshot["sequence"],
                    feedback_observed_monotonic_s=snapshot["observed_monotonic_s"],
                    audit_plan_started_monotonic_s=now, audit_plan_committed_monotonic_s=commit,
                    block_tokens=self.slot_spec.block_tokens, desired_blocks=desired,
                    gpu_blocks=selected, committed_blocks=sorted(self.committed),
                    requested_gpu_bytes=int(plan.gpu_bytes), requested_cpu_bytes=0,
                    status=dataclasses.asdict(status))
