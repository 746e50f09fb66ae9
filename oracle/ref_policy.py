"""Oracle: the reference's placement policy arithmetic, restated for the CPU.

TEST INFRASTRUCTURE ONLY -- never imported by the shipped package.

Each function names the reference lines it restates (paths are relative to the
reference project root).  Parity is pinned by ``tests/test_oracle_golden.py``
against fixtures generated from the unmodified reference modules.

One deliberate difference: the reference ranks blocks with
``np.argsort(-values)`` (experiments/slot_feedback.py:83), whose order among
equal timestamps depends on the numpy build.  The oracle uses a stable sort,
i.e. ties come out in ascending block id.  Inputs without ties give identical
results under both.
"""
from __future__ import annotations

import dataclasses
import math
from collections import deque

import numpy as np

INITIAL = (1 << 64) - 1          # experiments/cache_window.py:16


# --------------------------------------------------------------------------
# window policy
# --------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class WindowSpec:
    """Geometry of the bounded window (experiments/cache_window.py:19-29)."""
    allocation_bytes: int
    allocation_count: int
    bytes_per_token: int
    width_tokens: int = 32768
    lookahead_tokens: int = 16384
    quantum_tokens: int = 8192
    min_update_seconds: float = 1.0
    idle_only: bool = True
    update_mode: str = "incremental"


def check_window_spec(s: WindowSpec) -> None:
    """Validation order and messages of experiments/cache_window.py:31-50."""
    for name in ("allocation_bytes", "allocation_count", "bytes_per_token",
                 "width_tokens", "lookahead_tokens", "quantum_tokens"):
        v = getattr(s, name)
        if type(v) is not int or v <= 0:
            raise ValueError(f"cache_window.{name} must be a positive integer")
    if s.lookahead_tokens >= s.width_tokens:
        raise ValueError("cache window must retain a trailing region")
    if (s.quantum_tokens * s.bytes_per_token) % 4096:
        raise ValueError("cache window quantum must be page aligned")
    if s.width_tokens % s.quantum_tokens or s.lookahead_tokens % s.quantum_tokens:
        raise ValueError("cache window dimensions must be multiples of the quantum")
    if s.width_tokens * s.bytes_per_token > s.allocation_bytes:
        raise ValueError("cache window exceeds each allocation")
    if not math.isfinite(s.min_update_seconds) or s.min_update_seconds < 0:
        raise ValueError("invalid cache window update interval")
    if type(s.idle_only) is not bool:
        raise ValueError("cache_window.idle_only must be boolean")
    if s.update_mode not in ("incremental", "initial_only", "full_cache"):
        raise ValueError("invalid cache_window.update_mode")


def window(s: WindowSpec, completed_tokens: float) -> tuple[int, int]:
    """Byte window for a completed-token count (experiments/cache_window.py:52-63).

    The division is carried out in float64 and rounded up with ``math.ceil``
    exactly as the reference does, so non-integral counters agree too.
    """
    if not math.isfinite(completed_tokens) or completed_tokens < 0:
        raise ValueError("invalid completed-token count")
    q = s.quantum_tokens
    wanted_end = max(s.width_tokens,
                     math.ceil((completed_tokens + s.lookahead_tokens) / q) * q)
    last_end = s.allocation_bytes // (q * s.bytes_per_token) * q
    end = min(wanted_end, last_end)
    return (end - s.width_tokens) * s.bytes_per_token, end * s.bytes_per_token


def interval_difference(a, b):
    """a minus b as at most two half-open pieces (experiments/cache_window.py:66-68)."""
    pieces = ((a[0], min(a[1], b[0])), (max(a[0], b[1]), a[1]))
    return [(lo, hi) for lo, hi in pieces if hi > lo]


def window_accounting(s: WindowSpec, allocations, old, new, *, full: bool, refresh: bool):
    """requested_gpu_bytes / requested_cpu_bytes (experiments/cache_window.py:122-131).

    ``allocations`` is the registry snapshot (dicts with ``bytes``)."""
    n = sum(1 for a in allocations if a["bytes"] == s.allocation_bytes)
    if full:
        gpu = sum(a["bytes"] for a in allocations if a["bytes"] != s.allocation_bytes)
        gpu += n * (new[1] - new[0])
        cpu = n * (s.allocation_bytes - new[1] + new[0])
    elif refresh:
        gpu = n * (new[1] - new[0])
        cpu = n * (s.allocation_bytes - new[1] + new[0])
    else:
        gpu = n * sum(hi - lo for lo, hi in interval_difference(new, old))
        cpu = n * sum(hi - lo for lo, hi in interval_difference(old, new))
    return gpu, cpu


# --------------------------------------------------------------------------
# slot metadata -> runs -> blocks
# --------------------------------------------------------------------------
def encode_runs(values):
    """Half-open runs of consecutive values, keeping order and repeats
    (experiments/kv_audit/kv_audit_probe.py:23-32)."""
    runs: list[list[int]] = []
    for v in values:
        v = int(v)
        if runs and runs[-1][1] == v:
            runs[-1][1] = v + 1
        else:
            runs.append([v, v + 1])
    return runs


class FeedbackState:
    """Per-slot generations and per-block version / last-read / last-write
    state (experiments/slot_feedback.py:10-96), without the file drop: the
    snapshot dict that the reference serialises is returned instead."""

    def __init__(self, block_tokens=256, publish_seconds=.05, pid=0):
        self.block_tokens = block_tokens
        self.publish_seconds = publish_seconds
        self.pid = pid
        self.epoch = 0
        self.sequence = -1
        self.last_publish = -float("inf")
        self.capacity = 0
        self.free_head = deque()
        self.last_snapshot = None

    def reset(self, capacity):
        """experiments/slot_feedback.py:25-33"""
        t = self.block_tokens
        self.capacity = capacity
        self.generations = np.zeros(capacity + 1, dtype=np.int32)
        count = (capacity + 1 + t - 1) // t
        self.versions = np.zeros(count, dtype=np.int32)
        self.read_seen = np.full(count, -float("inf"))
        self.write_seen = np.full(count, -float("inf"))
        self.free_head.clear()
        self.epoch += 1

    def blocks(self, ranges):
        """Blocks covered by slot runs, first-seen order, slot 0 excluded
        (experiments/slot_feedback.py:35-46)."""
        t = self.block_tokens
        out, seen = [], set()
        for begin, end in ranges:
            begin = max(1, begin)
            if begin >= end:
                continue
            if end > self.capacity + 1:
                raise AssertionError("slot beyond capacity")
            for blk in range(begin // t, (end - 1) // t + 1):
                if blk not in seen:
                    seen.add(blk)
                    out.append(blk)
        return out

    def consume(self, row):
        """experiments/slot_feedback.py:48-79"""
        kind, at = row["event"], row["monotonic_s"]
        self.sequence = row["sequence"]
        t = self.block_tokens
        if kind == "allocator_clear":
            self.reset(row["allocator_size"])
        elif kind == "alloc":
            if not self.capacity:
                self.reset(row["allocator_size"])
            allocated = row["slot_runs"]
            for begin, end in allocated:
                begin = max(begin, 1)
                if end > begin:
                    self.generations[begin:end] += 1
            for blk in self.blocks(allocated):
                lo = blk * t
                self.versions[blk] = self.generations[lo:lo + t].max()
                self.write_seen[blk] = at
            if "free_head_runs" in row:
                self.free_head = deque(s for a, b in row["free_head_runs"] for s in range(a, b))
            else:
                taken = {s for a, b in allocated for s in range(a, b)}
                self.free_head = deque(s for s in self.free_head if s not in taken)
        elif kind == "attention" and self.capacity:
            for blk in self.blocks(row["read_runs"]):
                self.read_seen[blk] = at
            for blk in self.blocks(row["write_runs"]):
                self.write_seen[blk] = at
        if self.capacity and at - self.last_publish >= self.publish_seconds:
            self.publish(at)

    def publish(self, at, published=None):
        """experiments/slot_feedback.py:81-96 (stable tie order, see module doc)."""
        def recent(values):
            order = np.argsort(-values, kind="stable")
            return [[int(i), float(values[i])] for i in order
                    if np.isfinite(values[i]) and at - values[i] <= 30]
        t = self.block_tokens
        free = list(dict.fromkeys(s // t for s in self.free_head))
        row = dict(version=1, pid=self.pid, epoch=self.epoch, sequence=self.sequence,
                   observed_monotonic_s=at,
                   published_monotonic_s=at if published is None else published,
                   capacity_tokens=self.capacity, block_tokens=t,
                   block_versions=self.versions.tolist(),
                   recent_reads=recent(self.read_seen),
                   recent_writes=recent(self.write_seen),
                   free_head_blocks=free)
        self.last_publish = at
        self.last_snapshot = row
        return row


# --------------------------------------------------------------------------
# block ranking and selection
# --------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class SlotSpec:
    """experiments/slot_placement.py:18-26"""
    block_tokens: int = 256
    lookahead_tokens: int = 4096
    min_update_seconds: float = .25
    max_blocks_per_update: int = 4
    active_seconds: float = 2.0
    refresh_seconds: float = 10.0
    max_feedback_lag_seconds: float = 1.0


def check_slot_spec(s: SlotSpec) -> None:
    """experiments/slot_placement.py:28-34 (the reference raises ValueError(key))."""
    for key in ("block_tokens", "lookahead_tokens", "max_blocks_per_update"):
        v = getattr(s, key)
        if type(v) is not int or v <= 0:
            raise ValueError(key)
    for key in ("min_update_seconds", "active_seconds", "refresh_seconds",
                "max_feedback_lag_seconds"):
        v = getattr(s, key)
        if not math.isfinite(v) or v <= 0:
            raise ValueError(key)


def target_blocks(snapshot, spec: SlotSpec, budget: int, now: float):
    """Active reads, active writes, free-list head, then history by recency;
    first occurrence wins; cut at the budget (experiments/slot_placement.py:37-44)."""
    reads, writes = snapshot["recent_reads"], snapshot["recent_writes"]
    live_r = [b for b, t in reads if now - t <= spec.active_seconds]
    live_w = [b for b, t in writes if now - t <= spec.active_seconds]
    history = [b for b, _ in sorted(reads + writes, key=lambda p: -p[1])]
    order = list(dict.fromkeys(live_r + live_w + list(snapshot["free_head_blocks"]) + history))
    return order[:budget]


def encode_mask(blocks) -> str:
    """Lower-case hex of OR(1 << b), no prefix (experiments/slot_placement.py:47-51)."""
    m = 0
    for b in blocks:
        m |= 1 << b
    return format(m, "x")


def choose(snapshot, spec: SlotSpec, budget: int, committed: dict, now: float):
    """desired, selected (experiments/slot_placement.py:83-94).

    ``committed`` maps block -> (version, commit_time)."""
    desired = target_blocks(snapshot, spec, budget, now)
    versions = snapshot["block_versions"]
    events = snapshot["recent_reads"] + snapshot["recent_writes"]
    todo = []
    for blk in desired:
        old = committed.get(blk)
        if (old is None or old[0] != versions[blk]
                or (now - old[1] >= spec.refresh_seconds
                    and any(i == blk and now - t <= spec.active_seconds for i, t in events))):
            todo.append(blk)
    return desired, todo[:spec.max_blocks_per_update]


def retain_committed(committed: dict, desired, selected, versions, commit_time: float):
    """Bookkeeping after an accepted plan (experiments/slot_placement.py:150-153)."""
    want = set(desired)
    kept = {b: v for b, v in committed.items() if b in want}
    for b in selected:
        kept[b] = (versions[b], commit_time)
    return kept


def slot_plan_budget(w: WindowSpec, s: SlotSpec) -> int:
    """experiments/slot_placement.py:60-64"""
    budget = w.width_tokens // s.block_tokens
    if not budget or w.width_tokens % s.block_tokens:
        raise ValueError("KV budget must be divisible by block_tokens")
    if (s.block_tokens * w.bytes_per_token) % 4096:
        raise ValueError("slot blocks must be page aligned")
    return budget


def covered_bytes(selected, block_bytes: int, allocation_bytes: int, n_cache: int) -> int:
    """requested_gpu_bytes of a block plan (experiments/slot_placement.py:154)."""
    return sum(min(block_bytes, allocation_bytes - b * block_bytes) for b in selected) * n_cache
