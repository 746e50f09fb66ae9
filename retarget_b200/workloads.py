"""Seeded synthetic inputs for the placement planner.

The reference evaluates on live serving traffic that cannot be reproduced
offline, so every workload here is synthetic: a paged KV pool whose 16-slot
pages are handed out from a seeded random permutation, request lengths drawn
from a clipped log-normal, and (for the sparse case) attention-touched slot
sets made of the newest 128 slots plus 2048 Zipf-distributed history draws.
All randomness comes from ``numpy.random.default_rng(seed)``.

Slot ids follow the serving engine's convention (the reference's
experiments/slot_feedback.py:27-28,39): valid ids are ``1..capacity`` and id 0
is a reserved padding slot, so page 0 is never handed out.
"""
from __future__ import annotations

import dataclasses
from collections import deque

import numpy as np

PAGE_SLOTS = 16
UVM_BLOCK = 2 << 20


@dataclasses.dataclass(frozen=True)
class Layout:
    """KV geometry: ``2*layers`` equally sized managed buffers (all K buffers
    first, then all V buffers -- the order the serving engine allocates them)."""
    layers: int
    bytes_per_slot: int
    pool_slots: int
    block_bytes: int = UVM_BLOCK
    shared_bitmap: bool = True     # one bitmap for all layers (False: one per layer)

    @property
    def alloc_bytes(self) -> int:
        return self.pool_slots * self.bytes_per_slot

    @property
    def n_buffers(self) -> int:
        return 2 * self.layers

    @property
    def block_tokens(self) -> int:
        return self.block_bytes // self.bytes_per_slot

    @property
    def n_blocks(self) -> int:
        return -(-self.alloc_bytes // self.block_bytes)

    @property
    def capacity(self) -> int:
        return self.pool_slots - 1

    @property
    def n_groups(self) -> int:
        return 1 if self.shared_bitmap else self.layers

    def buffer_group(self) -> np.ndarray:
        """Bitmap index of every buffer in registry order."""
        if self.shared_bitmap:
            return np.zeros(self.n_buffers, dtype=np.uint32)
        return np.tile(np.arange(self.layers, dtype=np.uint32), 2)


class PagePool:
    """FIFO free list of 16-slot pages, seeded order, page 0 withheld."""

    def __init__(self, pool_slots: int, rng: np.random.Generator, shuffle: bool = True):
        pages = pool_slots // PAGE_SLOTS
        # shuffle=False: pages go out in address order, the way a freshly started
        # allocator hands them out (the live set is then a region that moves
        # through the pool, which is what a bounded window can follow)
        order = rng.permutation(pages) if shuffle else np.arange(pages)
        self.free = deque(int(p) for p in order if p != 0)

    def take(self, n_pages: int) -> list[int]:
        n = min(n_pages, len(self.free))
        return [self.free.popleft() for _ in range(n)]

    def give(self, pages) -> None:
        self.free.extend(int(p) for p in pages)


def request_lengths(rng, count, median, sigma=0.8, lo=128, hi=8192) -> np.ndarray:
    raw = rng.lognormal(np.log(median), sigma, size=count)
    return np.clip(np.rint(raw), lo, hi).astype(np.int64)


def page_slots(pages, length) -> np.ndarray:
    """Slot ids of the first ``length`` tokens stored in ``pages``."""
    if length == 0:
        return np.zeros(0, dtype=np.int64)
    p = np.asarray(pages, dtype=np.int64)
    return (p[:, None] * PAGE_SLOTS + np.arange(PAGE_SLOTS, dtype=np.int64)).reshape(-1)[:length]


def admit(pool: PagePool, lengths) -> list[np.ndarray]:
    """Give each request its pages in arrival order; a request that does not
    fit is cut to the pages that remain (possibly to nothing)."""
    out = []
    for n in lengths:
        pages = pool.take(-(-int(n) // PAGE_SLOTS))
        out.append(page_slots(pages, min(int(n), len(pages) * PAGE_SLOTS)))
    return out


@dataclasses.dataclass
class SlotBatch:
    """Flat slot indices in CSR form: group g owns
    ``slots[group_off[g]:group_off[g+1]]`` and request r of the whole batch owns
    ``slots[req_off[r]:req_off[r+1]]`` (requests never straddle groups)."""
    layout: Layout
    slots: np.ndarray          # int64
    group_off: np.ndarray      # int64 [G+1]
    req_off: np.ndarray        # int64 [R_total+1]
    budget_blocks: int
    name: str = ""

    @property
    def n_idx(self) -> int:
        return int(self.slots.shape[0])


def _dense_batch(layout, per_request, budget, name):
    lens = np.array([len(x) for x in per_request], dtype=np.int64)
    slots = np.concatenate(per_request) if per_request else np.zeros(0, np.int64)
    req_off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    return SlotBatch(layout, slots.astype(np.int64), np.array([0, len(slots)], np.int64),
                     req_off, budget, name)


def full_refresh(seed=0, *, layers=40, pool_slots=65536, bytes_per_slot=2048,
                 requests=64, median=1024, hi=8192, budget_frac=0.25) -> SlotBatch:
    """Dense decode read set: every cached slot of every live request, one
    bitmap shared by all layers."""
    rng = np.random.default_rng(seed)
    layout = Layout(layers, bytes_per_slot, pool_slots)
    pool = PagePool(pool_slots, rng)
    per_request = admit(pool, request_lengths(rng, requests, median, hi=hi))
    return _dense_batch(layout, per_request, int(layout.n_blocks * budget_frac),
                        f"full-refresh L{layers} R{requests} S{pool_slots}")


def tp_shard(seed=0, *, layers=48, pool_slots=262144, requests=256, median=4096,
             hi=32768, budget_frac=0.25) -> SlotBatch:
    """One tensor-parallel rank's view: one KV head (256 B per slot), the slot
    table is identical on every rank."""
    return dataclasses.replace(
        full_refresh(seed, layers=layers, pool_slots=pool_slots, bytes_per_slot=256,
                     requests=requests, median=median, hi=hi, budget_frac=budget_frac),
        name=f"tp-shard L{layers} R{requests} S{pool_slots}")


def bounded_zipf_cdf(n: int, s: float) -> np.ndarray:
    w = np.arange(1, n + 1, dtype=np.float64) ** (-s)
    c = np.cumsum(w)
    return c / c[-1]


def sparse_feedback(seed=0, *, layers=40, pool_slots=131072, bytes_per_slot=2048,
                    requests=128, median=512, recent=128, draws=2048, zipf_s=1.1,
                    budget_frac=0.15) -> SlotBatch:
    """Per (layer, request) touched sets: the newest ``recent`` slots followed
    by ``draws`` positions sampled Zipf(s) by age (rank 1 = newest token,
    support cut at the request's history).  One bitmap per layer."""
    rng = np.random.default_rng(seed)
    layout = Layout(layers, bytes_per_slot, pool_slots, shared_bitmap=False)
    pool = PagePool(pool_slots, rng)
    tables = admit(pool, request_lengths(rng, requests, median))
    cdfs = [bounded_zipf_cdf(len(t), zipf_s) if len(t) else None for t in tables]
    chunks, lens = [], []
    for _layer in range(layers):
        for t, cdf in zip(tables, cdfs):
            n = len(t)
            if n == 0:
                lens.append(0)
                continue
            tail = t[max(0, n - recent):]
            age = np.searchsorted(cdf, rng.random(draws), side="left") + 1
            picks = t[n - np.minimum(age, n)]
            chunks.append(tail)
            chunks.append(picks)
            lens.append(len(tail) + draws)
    slots = np.concatenate(chunks).astype(np.int64)
    req_off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    group_off = req_off[::requests].copy()
    return SlotBatch(layout, slots, group_off, req_off,
                     int(layout.n_blocks * budget_frac),
                     f"sparse-feedback L{layers} R{requests} S{pool_slots}")


def target_step(seed=0) -> SlotBatch:
    """The headline decode step: 40 layers, 256 requests, 262,144-slot pool,
    sparse per-layer touched sets (about 178 MB of int64 indices)."""
    b = sparse_feedback(seed, layers=40, pool_slots=262144, requests=256, median=512)
    b.name = "target-step L40 R256 S262144 sparse"
    return b


def confine(batch: SlotBatch, blocks, tag: str) -> SlotBatch:
    """Move a batch onto a subset of the pool's blocks: block b of the original
    goes to ``blocks[b % len(blocks)]`` and every id keeps its offset inside
    the block.  Sizes, request structure and the repeat pattern of the ids are
    unchanged; only the set of touched blocks is."""
    lay = batch.layout
    T = lay.block_tokens
    table = np.asarray(list(blocks), dtype=np.int64)
    assert len(table) and table.max() < lay.n_blocks and batch.slots.min() >= 1
    s = batch.slots
    moved = np.maximum(table[(s // T) % len(table)] * T + s % T, 1)   # id 0 is the padding slot
    assert moved.max() <= lay.capacity
    return dataclasses.replace(batch, slots=moved, name=f"{batch.name}, {tag}")


def target_pair(kind: str = "moving"):
    """Two headline-sized steps that alternate in the benchmark.

    ``moving``      step A lives in the lower half of every buffer, step B in the
                    upper half: each plan evicts one run and adds one run per
                    buffer (160 ranges), the shape of the reference's incremental
                    window update
    ``steady``      both steps want the same blocks: after the first plan nothing
                    moves (0 ranges), the common case of consecutive decode steps
    ``fragmented``  step A touches only even blocks, step B only odd ones: every
                    plan replaces the whole budget in single-block runs
                    (2 x 38 x 80 = 6080 ranges), the most the tail can be asked for
    """
    a, b = target_step(0), target_step(1)
    nb = a.layout.n_blocks
    if kind == "steady":
        return a, b
    if kind == "moving":
        return (confine(a, range(0, nb // 2), "lower half"),
                confine(b, range(nb // 2, nb), "upper half"))
    if kind == "fragmented":
        return (confine(a, range(0, nb, 2), "even blocks"),
                confine(b, range(1, nb, 2), "odd blocks"))
    raise ValueError(kind)


# --------------------------------------------------------------------------
# incremental decode trace
# --------------------------------------------------------------------------
@dataclasses.dataclass
class TraceStep:
    """One decode step of the incremental trace."""
    alloc_slots: np.ndarray    # slots of pages handed out this step (alloc events)
    read_slots: np.ndarray     # all cached slots of the live batch (attention read)
    write_slots: np.ndarray    # the slot each live request writes this step
    completed_tokens: int      # cumulative prompt + generated tokens after the step
    live: int
    free_head: np.ndarray | None = None   # first 4096 free slots, sampled on even steps
    req_off: np.ndarray | None = None     # request r of the live batch owns read_slots[req_off[r]:req_off[r+1]]


def decode_trace(seed=0, *, steps=256, pool_slots=65536, arrival_rate=0.5, median=1024,
                 mean_output=256, initial_requests=0, shuffle_pages=True) -> list[TraceStep]:
    """Poisson arrivals, log-normal prompts, geometric output lengths; every
    live request appends one token per step and finished requests return their
    pages to the tail of the free list."""
    rng = np.random.default_rng(seed)
    pool = PagePool(pool_slots, rng, shuffle_pages)
    live: list[dict] = []
    completed = 0
    trace = []
    for step in range(steps):
        new_pages: list[int] = []
        arrivals = int(rng.poisson(arrival_rate)) + (initial_requests if step == 0 else 0)
        for _ in range(arrivals):
            prompt = int(request_lengths(rng, 1, median)[0])
            out_len = int(rng.geometric(1.0 / mean_output))
            pages = pool.take(-(-prompt // PAGE_SLOTS))
            if len(pages) * PAGE_SLOTS < prompt:      # pool exhausted: request is dropped
                pool.give(pages)
                continue
            new_pages += pages
            live.append(dict(pages=pages, length=prompt, left=out_len))
            completed += prompt
        writes = []
        for r in live:
            if r["length"] == len(r["pages"]) * PAGE_SLOTS:
                got = pool.take(1)
                if not got:
                    r["left"] = 0
                    continue
                r["pages"] += got
                new_pages += got
            r["length"] += 1
            r["left"] -= 1
            completed += 1
            writes.append(r["pages"][(r["length"] - 1) // PAGE_SLOTS] * PAGE_SLOTS
                          + (r["length"] - 1) % PAGE_SLOTS)
        reads = [page_slots(r["pages"], r["length"]) for r in live]
        trace.append(TraceStep(
            alloc_slots=page_slots(new_pages, len(new_pages) * PAGE_SLOTS),
            read_slots=np.concatenate(reads) if reads else np.zeros(0, np.int64),
            write_slots=np.array(writes, dtype=np.int64),
            completed_tokens=completed, live=len(live),
            req_off=np.concatenate([[0], np.cumsum([len(x) for x in reads])]).astype(np.int64),
            free_head=(page_slots(list(pool.free)[:4096 // PAGE_SLOTS], 4096)[:len(pool.free) * PAGE_SLOTS]
                       if step % 2 == 0 else None)))
        done = [r for r in live if r["left"] <= 0]
        live = [r for r in live if r["left"] > 0]
        for r in done:
            pool.give(r["pages"])
    return trace
