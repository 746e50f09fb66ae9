"""Slot-feedback state in GPU memory (``rt_feedback_*``).

``DeviceFeedback`` takes the serving engine's index tensors where they are --
on the device -- and keeps the state the reference's ``SlotFeedback``
(experiments/slot_feedback.py) rebuilds on the host from pinned copies.  It
serves both ways of planning:

* ``plan()`` ranks, selects and emits the byte ranges on the device;
* ``snapshot()`` returns the dictionary the reference publishes as a JSON file,
  so ``SlotPlacementController(snapshot_source=fb.snapshot)`` runs unchanged.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import pathlib
import time

import numpy as np

from . import capi
from .planner import DevicePlanner, _is_i32, _ptr

FREE_HEAD_MAX = 4096


class FeedbackPolicy(C.Structure):
    _fields_ = [("budget", C.c_uint32), ("max_blocks_per_update", C.c_uint32), ("flags", C.c_uint32),
                ("reserved", C.c_uint32), ("active_seconds", C.c_double), ("refresh_seconds", C.c_double)]


class StepIds(C.Structure):
    _fields_ = [("d_allocated", C.c_void_p), ("n_allocated", C.c_uint64), ("d_free_head", C.c_void_p),
                ("n_free", C.c_uint32), ("reserved", C.c_uint32), ("t_allocated", C.c_double),
                ("d_read", C.c_void_p), ("n_read", C.c_uint64), ("d_written", C.c_void_p),
                ("n_written", C.c_uint64), ("t_attention", C.c_double)]


def _bind():
    lib = capi.lib
    vp = C.c_void_p
    lib.rt_feedback_create.argtypes = [vp, C.POINTER(vp)]
    lib.rt_feedback_destroy.argtypes = [vp]
    lib.rt_feedback_reset.argtypes = [vp, vp]
    lib.rt_feedback_alloc.argtypes = [vp, vp, C.c_uint64, vp, C.c_uint32, C.c_double, vp]
    lib.rt_feedback_attention.argtypes = [vp, vp, C.c_uint64, vp, C.c_uint64, C.c_double, vp]
    lib.rt_feedback_alloc_i32.argtypes = lib.rt_feedback_alloc.argtypes
    lib.rt_feedback_attention_i32.argtypes = lib.rt_feedback_attention.argtypes
    lib.rt_feedback_snapshot.argtypes = [vp, vp, vp, vp, vp, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64),
                                         C.POINTER(C.c_uint64)]
    lib.rt_feedback_plan.argtypes = [vp, C.POINTER(FeedbackPolicy), C.c_double, C.c_double, vp, C.c_uint32,
                                     vp, vp]
    lib.rt_feedback_step.argtypes = [vp, C.POINTER(StepIds), C.POINTER(FeedbackPolicy), C.c_double, vp,
                                     C.c_uint32, vp, vp]
    lib.rt_feedback_step_i32.argtypes = lib.rt_feedback_step.argtypes
    return lib


class DeviceFeedback:
    def __init__(self, planner: DevicePlanner, pid: int | None = None):
        self.lib = _bind()
        self.planner = planner
        self.layout = planner.layout
        self.pid = os.getpid() if pid is None else pid
        handle = C.c_void_p()
        capi.check(self.lib.rt_feedback_create(planner._h, C.byref(handle)), "rt_feedback_create")
        self._h = handle
        self.sequence = -1
        self.at = -float("inf")

    def close(self):
        if getattr(self, "_h", None):
            self.lib.rt_feedback_destroy(self._h)
            self._h = None

    __del__ = close

    def _event(self, t):
        self.sequence += 1
        self.at = t

    def clear(self, t, stream=None):
        self._event(t)
        capi.check(self.lib.rt_feedback_reset(self._h, stream), "rt_feedback_reset")

    def free(self, t):
        """A `free` row: the state ignores it (experiments/slot_feedback.py:76-77),
        only the time of the last observation moves."""
        self._event(t)

    def alloc(self, d_slots, t, d_free_head=None, stream=None):
        self._event(t)
        n_free = 0 if d_free_head is None else min(int(d_free_head.numel()), FREE_HEAD_MAX)
        narrow = _is_i32(d_slots)
        if d_free_head is not None and _is_i32(d_free_head) != narrow:
            raise TypeError("the slot list and the free head of one event must have the same dtype")
        fn = self.lib.rt_feedback_alloc_i32 if narrow else self.lib.rt_feedback_alloc
        capi.check(fn(self._h, _ptr(d_slots), int(d_slots.numel()), _ptr(d_free_head),
                                              n_free, float(t), stream), "rt_feedback_alloc")

    def attention(self, d_read, d_write, t, stream=None):
        self._event(t)
        narrow = _is_i32(d_read)
        if _is_i32(d_write) != narrow:
            raise TypeError("the read and write lists of one event must have the same dtype")
        fn = self.lib.rt_feedback_attention_i32 if narrow else self.lib.rt_feedback_attention
        capi.check(fn(self._h, _ptr(d_read), int(d_read.numel()), _ptr(d_write),
                                                  int(d_write.numel()), float(t), stream), "rt_feedback_attention")

    def plan(self, now, *, budget, max_blocks_per_update, active_seconds, refresh_seconds, flags,
             d_out, d_result, stream=None):
        pol = FeedbackPolicy(budget, max_blocks_per_update, flags, 0, active_seconds, refresh_seconds)
        cap = d_out.numel() * d_out.element_size() // capi.RANGE_DTYPE.itemsize
        capi.check(self.lib.rt_feedback_plan(self._h, C.byref(pol), float(self.at), float(now), _ptr(d_out),
                                             cap, _ptr(d_result), stream), "rt_feedback_plan")

    def step(self, *, d_allocated, t_allocated, d_read, d_written, t_attention, now, budget,
             max_blocks_per_update, active_seconds, refresh_seconds, flags, d_out, d_result, d_free_head=None,
             stream=None):
        """One decode step in one launch: ``alloc`` (skipped when ``d_allocated`` is
        None), ``attention`` and ``plan``, with the results of the three calls in
        that order."""
        lists = [x for x in (d_allocated, d_free_head, d_read, d_written) if x is not None]
        narrow = _is_i32(d_read)
        if any(_is_i32(x) != narrow for x in lists):
            raise TypeError("the id lists of one step must have the same dtype")
        if d_allocated is not None:
            self._event(t_allocated)
        self._event(t_attention)
        n_free = 0 if d_free_head is None else min(int(d_free_head.numel()), FREE_HEAD_MAX)
        ids = StepIds(_ptr(d_allocated), 0 if d_allocated is None else int(d_allocated.numel()),
                      _ptr(d_free_head), n_free, 0, float(t_allocated), _ptr(d_read), int(d_read.numel()),
                      _ptr(d_written), int(d_written.numel()), float(t_attention))
        pol = FeedbackPolicy(budget, max_blocks_per_update, flags, 0, active_seconds, refresh_seconds)
        cap = d_out.numel() * d_out.element_size() // capi.RANGE_DTYPE.itemsize
        fn = self.lib.rt_feedback_step_i32 if narrow else self.lib.rt_feedback_step
        capi.check(fn(self._h, C.byref(ids), C.byref(pol), float(now), _ptr(d_out), cap, _ptr(d_result), stream),
                   "rt_feedback_step")

    def arrays(self):
        nb = self.layout.n_blocks
        versions = np.zeros(nb, np.int32)
        reads, writes = np.zeros(nb, np.float64), np.zeros(nb, np.float64)
        free = np.zeros(FREE_HEAD_MAX, np.int64)
        n_free, epoch, bad = C.c_uint32(), C.c_uint64(), C.c_uint64()
        capi.check(self.lib.rt_feedback_snapshot(self._h, _ptr(versions), _ptr(reads), _ptr(writes), _ptr(free),
                                                 C.byref(n_free), C.byref(epoch), C.byref(bad)),
                   "rt_feedback_snapshot")
        return versions, reads, writes, free[:n_free.value], epoch.value, bad.value

    def publish(self, directory, at=None):
        """Writes the snapshot where the reference's controller looks for it:
        ``<directory>/<pid>.json``, through ``.<pid>.tmp`` and a rename
        (experiments/slot_feedback.py:86-96)."""
        directory = pathlib.Path(directory)
        directory.mkdir(parents=True, exist_ok=True)
        row = self.snapshot()
        if at is not None:
            row["observed_monotonic_s"] = at
        row["published_monotonic_s"] = time.monotonic()
        tmp = directory / f".{self.pid}.tmp"
        tmp.write_text(json.dumps(row, separators=(",", ":")))
        tmp.replace(directory / f"{self.pid}.json")
        return row

    def snapshot(self, now=None):
        """The reference's snapshot document (experiments/slot_feedback.py:86-91);
        ties among equal stamps come out in ascending block id."""
        versions, reads, writes, free, epoch, _ = self.arrays()
        at = self.at
        t = self.layout.block_tokens

        def recent(values):
            order = np.argsort(-values, kind="stable")
            return [[int(i), float(values[i])] for i in order if np.isfinite(values[i]) and at - values[i] <= 30]
        return dict(version=1, pid=self.pid, epoch=int(epoch), sequence=self.sequence,
                    observed_monotonic_s=at, published_monotonic_s=at,
                    capacity_tokens=self.layout.capacity, block_tokens=t,
                    block_versions=versions.tolist(), recent_reads=recent(reads), recent_writes=recent(writes),
                    free_head_blocks=list(dict.fromkeys(int(x) // t for x in free)))
