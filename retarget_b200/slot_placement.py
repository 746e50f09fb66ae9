"""Slot-feedback block placement: the scheduler-facing controller.

Drop-in for the reference's experiments/slot_placement.py: ``SlotPlacementSpec``,
``target_blocks``, ``encode_mask`` and ``SlotPlacementController`` keep their
names, arguments, error behaviour, socket commands and result dictionaries.
The mask encoding and the budget rule are the native library's
(``rt_encode_mask``, ``rt_slot_budget``).

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
from .cache_window import CacheWindowController
from .control import ControlError


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
        for key in ("block_tokens", "lookahead_tokens", "max_blocks_per_update"):
            value = getattr(self, key)
            if type(value) is not int or value <= 0:
                raise ValueError(key)
        for key in ("min_update_seconds", "active_seconds", "refresh_seconds",
                    "max_feedback_lag_seconds"):
            value = getattr(self, key)
            if not math.isfinite(value) or value <= 0:
                raise ValueError(key)


def target_blocks(snapshot, spec, budget, now):
    """Recent reads, recent writes, free-list head, then everything by recency;
    first mention wins; cut at the budget (experiments/slot_placement.py:37-44)."""
    reads, writes = snapshot["recent_reads"], snapshot["recent_writes"]
    fresh = [b for b, t in reads if now - t <= spec.active_seconds]
    fresh += [b for b, t in writes if now - t <= spec.active_seconds]
    by_recency = [b for b, _ in sorted(reads + writes, key=lambda item: -item[1])]
    seen, ranked = set(), []
    for b in fresh + list(snapshot["free_head_blocks"]) + by_recency:
        if b not in seen:
            seen.add(b)
            ranked.append(b)
    return ranked[:budget]


def encode_mask(blocks) -> str:
    """experiments/slot_placement.py:47-51"""
    blocks = list(blocks)
    arr = (C.c_uint32 * max(1, len(blocks)))(*blocks)
    cap = (max(blocks) // 4 + 3) if blocks else 3
    buf = C.create_string_buffer(cap)
    capi.check(capi.lib.rt_encode_mask(arr, len(blocks), buf, cap), "rt_encode_mask")
    return buf.value.decode()


class SlotPlacementController(CacheWindowController):
    """experiments/slot_placement.py:55-162"""

    def __init__(self, cache_spec, slot_spec, pid, snapshot_source=None):
        super().__init__(cache_spec)
        self.slot_spec = slot_spec
        self.pid = pid
        self._source = snapshot_source
        if snapshot_source is None:
            self.feedback_path = Path(os.environ["RETARGET_SLOT_FEEDBACK_DIR"]) / f"{pid}.json"
        budget = C.c_uint64()
        status = capi.lib.rt_slot_budget(C.byref(cache_spec._struct()), slot_spec.block_tokens,
                                         C.byref(budget))
        if status:
            raise ValueError(capi.strerror(status))
        self.budget = budget.value
        self.committed = {}
        self.epoch = None
        self.last_attempt = -math.inf

    def snapshot(self, now):
        if self._source is not None:
            data = self._source(now)
            if data is None:
                return None
        else:
            try:
                data = json.loads(self.feedback_path.read_text())
            except FileNotFoundError:
                return None
        if data["pid"] != self.pid or data["block_tokens"] != self.slot_spec.block_tokens:
            raise ControlError("slot feedback identity or geometry mismatch")
        if data["published_monotonic_s"] - data["observed_monotonic_s"] > \
                self.slot_spec.max_feedback_lag_seconds:
            return None
        return data

    def choose(self, snapshot, now):
        spec = self.slot_spec
        desired = target_blocks(snapshot, spec, self.budget, now)
        versions = snapshot["block_versions"]
        active = {b for b, t in snapshot["recent_reads"] + snapshot["recent_writes"]
                  if now - t <= spec.active_seconds}
        todo = []
        for block in desired:
            held = self.committed.get(block)
            if (held is None or held[0] != versions[block]
                    or (now - held[1] >= spec.refresh_seconds and block in active)):
                todo.append(block)
        return desired, todo[:spec.max_blocks_per_update]

    def due(self, metrics, now):
        if now - self.last_attempt < self.slot_spec.min_update_seconds:
            return False
        snapshot = self.snapshot(now)
        if snapshot is None:
            return False
        if self.epoch != snapshot["epoch"]:
            return True
        return bool(self.choose(snapshot, now)[1])

    def update(self, uvm, metrics, now, *, initial=False):
        if initial:
            result = super().update(uvm, metrics, now, initial=True)
            snapshot = self.snapshot(time.monotonic())
            if snapshot is None:
                raise ControlError("slot feedback unavailable after model warmup")
            self.epoch = snapshot["epoch"]
            unit = self.slot_spec.block_tokens * self.spec.bytes_per_token
            stamp = time.monotonic()
            self.committed = {b: (snapshot["block_versions"][b], stamp)
                              for b in range(self.current[0] // unit, self.current[1] // unit)}
            result.update(placement_kind="slot_feedback", committed_blocks=sorted(self.committed),
                          block_tokens=self.slot_spec.block_tokens, feedback_epoch=self.epoch)
            return result
        self.last_attempt = now
        snapshot = self.snapshot(now)
        if snapshot is None:
            return None
        if self.epoch != snapshot["epoch"]:
            self.committed.clear()
            self.epoch = snapshot["epoch"]
        desired, selected = self.choose(snapshot, now)
        if not selected:
            return None
        generation, allocations = uvm._allocation_snapshot()
        cache = [a for a in allocations if a["bytes"] == self.spec.allocation_bytes]
        signature = tuple((a["id"], a["bytes"], a["device"]) for a in cache)
        if len(cache) != self.spec.allocation_count:
            raise ControlError("slot-placement cache geometry changed")
        if signature != self.signature:
            self.committed.clear()
            self.signature = signature
            desired, selected = self.choose(snapshot, now)
        block_bytes = self.slot_spec.block_tokens * self.spec.bytes_per_token
        command = (f"blocksv {generation} {self.spec.allocation_bytes} {self.spec.allocation_count} "
                   f"{block_bytes} {encode_mask(selected)}")
        uvm.wait_idle(timeout=600)
        reply = uvm.command(command)
        if not reply.get("ok"):
            self.committed.clear()
            raise ControlError(f"slot prefetch rejected: {reply}")
        try:
            status = uvm._wait_job(int(reply["job_id"]), timeout=600)
        except Exception:
            self.committed.clear()
            raise
        commit = time.monotonic()
        wanted = set(desired)
        kept = {b: v for b, v in self.committed.items() if b in wanted}
        for block in selected:
            kept[block] = (snapshot["block_versions"][block], commit)
        self.committed = kept
        self.last_update = commit
        covered = sum(min(block_bytes, self.spec.allocation_bytes - b * block_bytes)
                      for b in selected) * len(cache)
        return dict(initial=False, placement_kind="slot_feedback", update_mode="slot_feedback",
                    allocation_generation=generation, feedback_epoch=self.epoch,
                    feedback_sequence=snapshot["sequence"],
                    feedback_observed_monotonic_s=snapshot["observed_monotonic_s"],
                    audit_plan_started_monotonic_s=now, audit_plan_committed_monotonic_s=commit,
                    block_tokens=self.slot_spec.block_tokens, desired_blocks=desired,
                    gpu_blocks=selected, committed_blocks=sorted(self.committed),
                    requested_gpu_bytes=covered, requested_cpu_bytes=0,
                    status=dataclasses.asdict(status))
