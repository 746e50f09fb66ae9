"""Probe-side writer that keeps the slot metadata on the device.

The reference's probe (experiments/kv_audit/kv_audit_probe.py) hooks the serving
engine and hands every observation to ``Writer.submit(kind, tensors, **fields)``,
which copies the index tensors to pinned host memory, run-length encodes them
in a Python loop on a worker thread and feeds ``SlotFeedback``.  ``DeviceWriter``
has the same ``submit`` signature and the same event vocabulary, but hands the
tensors to the device-resident feedback state where they are: no copy, no
worker thread, no per-slot Python.  The snapshot file the controller reads is
written on the reference's schedule (at most every ``publish_seconds``).

Binding in the reference::

    # experiments/kv_audit/kv_audit_probe.py, in emit()
    -        _writer = Writer()
    +        from retarget_b200.probe import DeviceWriter
    +        _writer = DeviceWriter()

Geometry: the reference's probe asserts 80 buffers with 2048-byte slots
(kv_audit_probe.py:133); those are the defaults here and can be overridden by
keyword or by ``RETARGET_KV_BUFFERS`` / ``RETARGET_KV_SLOT_BYTES``.  A
``geometry`` event that disagrees raises, as the reference's assertions do.
"""
from __future__ import annotations

import os
import time

from .feedback import DeviceFeedback
from .planner import DevicePlanner
from .workloads import Layout


class DeviceWriter:
    def __init__(self, directory=None, *, pid=None, block_tokens=256, publish_seconds=.05, buffers=None,
                 slot_bytes=None, device=0, clock=time.monotonic):
        self.directory = directory if directory is not None else os.environ.get("RETARGET_SLOT_FEEDBACK_DIR")
        self.pid = os.getpid() if pid is None else pid
        self.block_tokens = block_tokens
        self.publish_seconds = publish_seconds
        self.buffers = int(buffers if buffers is not None else os.environ.get("RETARGET_KV_BUFFERS", 80))
        self.slot_bytes = int(slot_bytes if slot_bytes is not None
                              else os.environ.get("RETARGET_KV_SLOT_BYTES", 2048))
        self.device = device
        self.clock = clock
        self.sequence = 0
        self.last_attention = -float("inf")
        self.last_publish = -float("inf")
        self.last_snapshot = None
        self.capacity = 0
        self.planner = None
        self.feedback = None

    # ---- state ----------------------------------------------------------
    def _reset(self, capacity: int, at: float):
        """SlotFeedback.reset (experiments/slot_feedback.py:25-33): new capacity
        means new state; the same capacity clears it and starts a new epoch."""
        if self.feedback is not None and capacity == self.capacity:
            self.feedback.clear(at, self._stream())
            return
        epoch = 0
        if self.feedback is not None:
            epoch = self.feedback.arrays()[4]
            self.feedback.close()
            self.planner.close()
        self.capacity = capacity
        layout = Layout(max(self.buffers // 2, 1), self.slot_bytes, capacity + 1,
                        self.block_tokens * self.slot_bytes)
        self.planner = DevicePlanner(layout, self.device)
        self.feedback = DeviceFeedback(self.planner, pid=self.pid)
        for _ in range(epoch):          # epochs keep counting across a change of capacity
            self.feedback.clear(at, self._stream())

    def _stream(self):
        import torch
        return torch.cuda.current_stream().cuda_stream

    @staticmethod
    def _check(tensors):
        for key, value in (tensors or {}).items():
            if value is not None:
                assert value.ndim == 1 and value.is_contiguous(), (key, tuple(value.shape))

    # ---- the probe's entry point -----------------------------------------
    def submit(self, kind, tensors=None, **fields):
        """Same contract as the reference's Writer.submit (kv_audit_probe.py:54-80):
        1-D contiguous device tensors by name, plus the event's scalar fields."""
        start = self.clock()
        # without an audit log attention metadata is sampled; allocator events stay exact
        if kind == "attention":
            if start - self.last_attention < .05:
                return
            self.last_attention = start
        self._check(tensors)
        tensors = tensors or {}
        sequence = self.sequence
        self.sequence += 1
        if kind == "allocator_clear":
            self._reset(int(fields["allocator_size"]), start)
        elif kind == "alloc":
            if not self.capacity:
                self._reset(int(fields["allocator_size"]), start)
            self.feedback.alloc(tensors["slot"], start, tensors.get("free_head"), self._stream())
        elif kind == "attention" and self.capacity:
            read, write = tensors.get("read"), tensors.get("write")
            if read is not None and write is not None and read.dtype != write.dtype:
                # kv_indices and out_cache_loc differ in width: one call per list, same stamp
                self.feedback.attention(read, read[:0], start, self._stream())
                self.feedback.attention(write[:0], write, start, self._stream())
            else:
                read = read if read is not None else write[:0]
                write = write if write is not None else read[:0]
                self.feedback.attention(read, write, start, self._stream())
        elif kind == "geometry":
            self._check_geometry(fields)
        # 'free' proves nothing about drained GPU work and is ignored (slot_feedback.py:76-77)
        if self.feedback is not None:
            self.feedback.sequence = sequence
            self.feedback.at = start
        if self.capacity and self.directory and start - self.last_publish >= self.publish_seconds:
            self.publish(start)

    def _check_geometry(self, fields):
        entries = fields.get("allocations") or []
        if len(entries) != self.buffers or any(e["slot_bytes"] != self.slot_bytes for e in entries):
            raise AssertionError(f"KV geometry differs from the configured {self.buffers} buffers of "
                                 f"{self.slot_bytes}-byte slots")
        if self.capacity and int(fields.get("allocator_size", self.capacity)) != self.capacity:
            raise AssertionError("allocator size changed without an allocator_clear event")

    def publish(self, at):
        self.last_snapshot = self.feedback.publish(self.directory, at)
        self.last_publish = at
        return self.last_snapshot

    def close(self):
        if self.feedback is not None:
            self.feedback.close()
            self.planner.close()
            self.feedback = self.planner = None
