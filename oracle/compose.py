"""Oracle: how the reference functions are chained into a per-step plan.

TEST INFRASTRUCTURE ONLY -- never imported by the shipped package.

The reference plans one mask for all layers from sampled events; the planner
under test generalises that to one bitmap per group of buffers and adds an
optional eviction phase.  This file freezes that glue so both sides of a
parity test run the same recipe:

* a step's slot indices are run-length encoded per request
  (``encode_runs``), turned into blocks (``FeedbackState.blocks``) and stamped
  as one attention read at a single time; ``publish`` -> ``target_blocks``
  ranks them and cuts at the budget (ties: ascending block id);
* ``choose`` keeps the desired blocks that are not yet committed, with
  ``max_blocks_per_update`` set to the budget;
* the chosen blocks go through ``encode_mask`` and the ``blocksv`` expansion
  over the group's buffers (destination: the GPU);
* GLUE (no reference counterpart): with ``evict=True`` the committed blocks
  that are no longer desired are expanded the same way with destination CPU
  and are listed before every GPU range, mirroring the CPU-before-GPU phase
  order of the window commands;
* afterwards the committed set of a group equals its desired set -- unless
  nothing of the group moved, in which case its record is left as it was, as
  the reference's controller returns early when nothing was selected.
"""
from __future__ import annotations

import numpy as np

from . import ref_policy as rp
from . import uvm_expand as ux

T_NOW = 1.0   # the single event time used for one-event plans


def registry_for(layout, device=0, first_id=1, extra=()):
    """Registry as the preload library would hold it: cache buffers in
    allocation order, optional non-cache allocations after them."""
    reg = [dict(id=first_id + j, bytes=layout.alloc_bytes, device=device, concurrent=1)
           for j in range(layout.n_buffers)]
    nxt = first_id + layout.n_buffers
    for k, nbytes in enumerate(extra):
        reg.append(dict(id=nxt + k, bytes=int(nbytes), device=device, concurrent=1))
    return reg


def group_blocks_literal(slots, req_off, layout):
    """Touched blocks of one group, through the reference functions, in
    first-seen order."""
    fb = rp.FeedbackState(block_tokens=layout.block_tokens)
    fb.reset(layout.capacity)
    runs = []
    for r in range(len(req_off) - 1):
        runs += rp.encode_runs(slots[req_off[r]:req_off[r + 1]].tolist())
    fb.consume(dict(event="attention", monotonic_s=T_NOW, sequence=0,
                    read_runs=runs, write_runs=[]))
    return fb


def touched_blocks(slots, layout):
    """Ascending block ids touched by ``slots`` (all within 1..capacity or below
    1), through the restated reference functions: encode_runs -> blocks."""
    fb = rp.FeedbackState(block_tokens=layout.block_tokens)
    fb.reset(layout.capacity)
    return sorted(fb.blocks(rp.encode_runs(np.asarray(slots).tolist())))


def group_blocks_fast(slots, layout):
    """Same set as ``group_blocks_literal`` (ascending), vectorised; used only
    where the literal path would take minutes."""
    s = np.asarray(slots)
    if np.any(s > layout.capacity):
        raise AssertionError("slot beyond capacity")
    s = s[s >= 1]
    return np.unique(s // layout.block_tokens).tolist()


def _runs_of(blocks):
    """Sorted block ids -> [(begin, end)) runs."""
    out = []
    for b in sorted(blocks):
        if out and out[-1][1] == b:
            out[-1][1] = b + 1
        else:
            out.append([b, b + 1])
    return out


def plan_step(batch, resident, *, evict=True, literal=True, device=0):
    """One planning step over every group.

    ``resident`` is a list (one per group) of sets of committed block ids and
    is updated in place.  Returns ``(ranges, info)`` with ranges as
    ``(buffer_index, dst, offset, bytes)`` in emission order (dst -1 = CPU)."""
    lay = batch.layout
    spec = rp.SlotSpec(block_tokens=lay.block_tokens, max_blocks_per_update=max(batch.budget_blocks, 1))
    groups = lay.buffer_group()
    reg = registry_for(lay, device)
    U = lay.block_bytes
    add_sets, evict_sets = [], []
    for g in range(lay.n_groups):
        lo, hi = int(batch.group_off[g]), int(batch.group_off[g + 1])
        if literal:
            ro = batch.req_off
            k0, k1 = np.searchsorted(ro, lo, "left"), np.searchsorted(ro, hi, "right")
            ro_g = ro[k0:k1] - lo
            if len(ro_g) == 0 or ro_g[0] != 0:
                ro_g = np.concatenate([[0], ro_g])
            if ro_g[-1] != hi - lo:
                ro_g = np.concatenate([ro_g, [hi - lo]])
            fb = group_blocks_literal(batch.slots[lo:hi], ro_g, lay)
            snap = fb.publish(T_NOW)
        else:
            blocks = group_blocks_fast(batch.slots[lo:hi], lay)
            snap = dict(recent_reads=[[b, T_NOW] for b in blocks], recent_writes=[],
                        free_head_blocks=[], block_versions=[0] * (lay.capacity // lay.block_tokens + 1))
        committed = {b: (0, T_NOW) for b in resident[g]}
        desired, selected = rp.choose(snap, spec, batch.budget_blocks, committed, T_NOW)
        gone = set(resident[g]) - set(desired) if evict else set()
        add_sets.append(set(selected))
        evict_sets.append(gone)
        if selected or gone:
            # retained = committed & desired, plus what was sent (experiments/slot_placement.py:150-153)
            resident[g] = set(desired)
        # else: nothing moves and the controller returns before it touches
        # `committed` (experiments/slot_placement.py:131-132)
    out = []
    for phase, sets, dst in ((0, evict_sets, ux.CPU), (1, add_sets, device)):
        for j in range(lay.n_buffers):
            chosen = sets[groups[j]]
            if not chosen:
                continue
            one = [dict(reg[j])]
            got = ux.expand_blocks(one, 0, gen=0, alloc_bytes=lay.alloc_bytes, count=1,
                                   block_bytes=U, mask=rp.encode_mask(chosen))
            out += [(j, dst, off, n) for _, off, n, _ in got]
    info = dict(blocks_added=sum(len(s) for s in add_sets),
                blocks_evicted=sum(len(s) for s in evict_sets))
    return out, info


def window_blocks(lo, hi, block_bytes):
    """Block ids covered by a block-aligned byte window."""
    assert lo % block_bytes == 0 and (hi % block_bytes == 0)
    return set(range(lo // block_bytes, hi // block_bytes))


def window_step(spec, layout, completed, old, *, full=False, refresh=False, device=0, extra=()):
    """Counter-driven window plan: window() -> windowv/windowfullv expansion.
    ``old`` is the previous window or None.  Ranges come back as
    ``(buffer_index, dst, offset, bytes)``; non-cache allocations (``extra``)
    are numbered after the cache buffers."""
    new = rp.window(spec, completed)
    reg = registry_for(layout, device, extra=extra)
    first = old is None or full
    o = (rp.INITIAL, rp.INITIAL) if first else old
    got = ux.expand_window(reg, 0, gen=0, alloc_bytes=spec.allocation_bytes,
                           count=spec.allocation_count, old=o, new=new,
                           full_refresh=refresh and not first)
    ids = {a["id"]: k for k, a in enumerate(reg)}
    return new, [(ids[i], dst, off, n) for i, off, n, dst in got]


class FeedbackSession:
    """The reference's event-driven slot path on the CPU: SlotFeedback state ->
    publish -> target_blocks -> choose -> blocksv, with the controller's
    committed bookkeeping (commit time = planning time) and the eviction glue."""

    def __init__(self, layout, spec: rp.SlotSpec, budget: int, *, evict=True, device=0):
        assert layout.n_groups == 1
        self.layout, self.spec, self.budget, self.evict, self.device = layout, spec, budget, evict, device
        self.fb = rp.FeedbackState(block_tokens=layout.block_tokens, publish_seconds=1e18)
        self.fb.reset(layout.capacity)
        self.committed = {}
        self.sequence = 0
        self.at = -float("inf")
        self.reg = registry_for(layout, device)

    def _row(self, kind, t, **fields):
        self.sequence += 1
        self.at = t
        return dict(event=kind, monotonic_s=t, sequence=self.sequence, **fields)

    def clear(self, t):
        self.fb.consume(self._row("allocator_clear", t, allocator_size=self.layout.capacity))
        self.committed = {}

    def alloc(self, slots, free_head, t):
        row = self._row("alloc", t, slot_runs=rp.encode_runs(np.asarray(slots).tolist()),
                        allocator_size=self.layout.capacity)
        if free_head is not None:
            row["free_head_runs"] = rp.encode_runs(np.asarray(free_head).tolist())
        self.fb.consume(row)

    def free(self, slots, t):
        """A `free` row: ignored by the state (experiments/slot_feedback.py:76-77),
        but it moves the time of the last observation."""
        self.fb.consume(self._row("free", t, slot_runs=rp.encode_runs(np.asarray(slots).tolist())))

    def attention(self, read, write, t):
        self.fb.consume(self._row("attention", t, read_runs=rp.encode_runs(np.asarray(read).tolist()),
                                  write_runs=rp.encode_runs(np.asarray(write).tolist())))

    def snapshot(self):
        return self.fb.publish(self.at)

    def plan(self, now):
        lay = self.layout
        snap = self.snapshot()
        desired, selected = rp.choose(snap, self.spec, self.budget, self.committed, now)
        evicted = (set(self.committed) - set(desired)) if self.evict else set()
        if not selected and not evicted:
            # the controller returns before it touches `committed`
            # (experiments/slot_placement.py:131-132): a committed block that is
            # not desired right now stays on record
            return [], dict(desired=desired, selected=[], evicted=[], committed=sorted(self.committed))
        self.committed = rp.retain_committed(self.committed, desired, selected, snap["block_versions"], now)
        out = []
        for chosen, dst in ((evicted, ux.CPU), (set(selected), self.device)):
            if not chosen:
                continue
            for j in range(lay.n_buffers):
                got = ux.expand_blocks([dict(self.reg[j])], 0, gen=0, alloc_bytes=lay.alloc_bytes, count=1,
                                       block_bytes=lay.block_bytes, mask=rp.encode_mask(chosen))
                out += [(j, dst, off, n) for _, off, n, _ in got]
        return out, dict(desired=desired, selected=selected, evicted=sorted(evicted),
                         committed=sorted(self.committed))
