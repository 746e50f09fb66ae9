"""The three oracle forms agree: the literal chain of restated reference
functions, its vectorised shortcut, and the C restatement used for full-size
cases and as the timed CPU baseline."""
import dataclasses

import numpy as np
import pytest

from oracle import c_oracle, compose
from retarget_b200 import workloads


def _tuples(r):
    return [(int(x["buffer"]), int(x["dst"]), int(x["offset"]), int(x["bytes"])) for x in r]


def _batches():
    yield [workloads.full_refresh(0), workloads.full_refresh(1), workloads.full_refresh(0)]
    yield [workloads.sparse_feedback(s, layers=3, requests=12) for s in (0, 1, 2)]
    yield [workloads.tp_shard(s, requests=40) for s in (0, 1)]
    rng = np.random.default_rng(3)
    lay = workloads.Layout(2, 2048, 6001, 12288, False)      # 6 slots per block, partial tail
    seq = []
    for k in range(4):
        lens = rng.integers(0, 900, 6)
        slots = rng.integers(-3, lay.capacity + 1, int(lens.sum())).astype(np.int64)
        off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        seq.append(workloads.SlotBatch(lay, slots, off[::3].copy(), off, 30 + k))
    yield seq


@pytest.mark.parametrize("evict", [True, False])
def test_literal_fast_and_c_oracles_agree(evict):
    for seq in _batches():
        lay = seq[0].layout
        r_lit = [set() for _ in range(lay.n_groups)]
        r_fast = [set() for _ in range(lay.n_groups)]
        co = c_oracle.COracle(lay)
        for b in seq:
            want = compose.plan_step(b, r_lit, evict=evict, literal=True)
            assert compose.plan_step(b, r_fast, evict=evict, literal=False) == want
            for threads in (1, 3):
                if threads == 3:
                    co.resident[:] = saved
                saved = co.resident.copy()
                got, invalid = co.step(b.slots, b.group_off, b.budget_blocks, evict, threads)
                assert _tuples(got) == want[0] and invalid == 0
            assert co.resident_sets() == r_lit == r_fast


def test_three_oracle_forms_agree_at_a_million_ids():
    """8 layers x 64 requests x 2176 ids = 1.1 M ids, two steps that move blocks:
    the Python chain (one loop iteration per id, as the reference has it), the
    vectorised shortcut and the C chain give the same ranges and records.  The
    C chain is what the full-size GPU tests compare with."""
    nb = workloads.sparse_feedback(0, layers=8, requests=64).layout.n_blocks
    seq = [workloads.confine(workloads.sparse_feedback(0, layers=8, requests=64), range(0, nb, 2), "even"),
           workloads.confine(workloads.sparse_feedback(1, layers=8, requests=64), range(1, nb, 2), "odd")]
    assert seq[0].n_idx == 8 * 64 * 2176 > 1_000_000
    lay = seq[0].layout
    r_lit, r_fast = ([set() for _ in range(lay.n_groups)] for _ in range(2))
    co = c_oracle.COracle(lay)
    for b in seq:
        want = compose.plan_step(b, r_lit, evict=True, literal=True)
        assert compose.plan_step(b, r_fast, evict=True, literal=False) == want
        got, invalid = co.step(b.slots, b.group_off, b.budget_blocks, True)
        assert _tuples(got) == want[0] and invalid == 0 and len(got) > 0
        assert co.resident_sets() == r_lit == r_fast
    assert want[1]["blocks_evicted"] > 0


def test_slot_zero_and_negative_ids_are_dropped():
    lay = workloads.Layout(1, 2048, 4096)
    slots = np.array([0, -1, 0, 1, 2, 3, -9], dtype=np.int64)
    off = np.array([0, 7], dtype=np.int64)
    b = workloads.SlotBatch(lay, slots, off, off, 2)
    res = [set()]
    out, _ = compose.plan_step(b, res)
    assert res == [{0}] and len(out) == 2
    empty = dataclasses.replace(b, slots=np.array([0, -4], dtype=np.int64), group_off=np.array([0, 2]),
                                req_off=np.array([0, 2]))
    out, info = compose.plan_step(empty, res)
    assert res == [set()] and info["blocks_evicted"] == 1 and all(r[1] == -1 for r in out)


def test_slot_above_capacity_is_an_error_in_the_oracle():
    lay = workloads.Layout(1, 2048, 4096)
    off = np.array([0, 1], dtype=np.int64)
    b = workloads.SlotBatch(lay, np.array([4096], dtype=np.int64), off, off, 2)
    with pytest.raises(AssertionError):
        compose.plan_step(b, [set()])
    co = c_oracle.COracle(lay)
    _, invalid = co.step(b.slots, b.group_off, 2)
    assert invalid == 1


def test_workload_shapes_match_the_stated_configs():
    b = workloads.full_refresh(0)
    assert (b.layout.n_buffers, b.layout.alloc_bytes, b.layout.n_blocks, b.budget_blocks) == \
        (80, 128 << 20, 64, 16)
    assert b.slots.min() >= 16 and b.slots.max() <= b.layout.capacity
    t = workloads.tp_shard(0)
    assert (t.layout.n_buffers, t.layout.alloc_bytes, t.layout.n_blocks, t.layout.block_tokens) == \
        (96, 64 << 20, 32, 8192)
    s = workloads.sparse_feedback(0, layers=2, requests=8)
    assert s.layout.n_groups == 2 and s.n_idx == 2 * 8 * 2176 and s.budget_blocks == 19
    trace = workloads.decode_trace(0, steps=40)
    assert len(trace) == 40 and trace[-1].completed_tokens > 0
    assert workloads.full_refresh(0).slots.tobytes() == b.slots.tobytes()      # seeded


def test_benchmark_pairs_move_what_they_say():
    """The alternating pairs the benchmark times, through the vectorised and the
    C oracle: 160 ranges per step when the halves alternate, 6080 single-block
    ranges when even and odd blocks do, none once the steady pair has settled."""
    expected = {"moving": 160, "fragmented": 6080, "steady": 0}
    for kind, ranges in expected.items():
        a, b = workloads.target_pair(kind)
        assert a.n_idx == b.n_idx == 22_282_240 and a.layout.n_groups == 40
        assert a.slots.min() >= 1 and a.slots.max() <= a.layout.capacity
        resident = [set() for _ in range(a.layout.n_groups)]
        co = c_oracle.COracle(a.layout)
        for step, batch in enumerate((a, b, a)):
            want, info = compose.plan_step(batch, resident, literal=False)
            got, invalid = co.step(batch.slots, batch.group_off, batch.budget_blocks, True, 4)
            assert _tuples(got) == want and invalid == 0
            if step:
                assert len(want) == ranges, (kind, step)
                if ranges:
                    assert info["blocks_added"] == info["blocks_evicted"] == 40 * 38
