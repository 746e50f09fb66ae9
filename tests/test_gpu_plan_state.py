"""GPU: what the planner's state is after a step that could not be delivered.

A plan that overflows the caller's range buffer, or whose slot ids fall outside
the pool, must leave the resident bitmaps as they were -- the ranges were never
executed, so they must not count as resident on the next step (the reference
drops its record on any failure, experiments/slot_placement.py:140-147, and
checks the slot range before it stamps anything, experiments/slot_feedback.py:42).
Also here: a bitmap whose plan moves nothing keeps its record
(experiments/slot_placement.py:131-132)."""
import numpy as np
import pytest

from oracle import compose
from oracle import ref_policy as rp
from retarget_b200 import capi, workloads
from retarget_b200.feedback import DeviceFeedback
from retarget_b200.planner import (DevicePlanner, ranges_from_tensor, ranges_to_tuples,
                                   result_from_tensor)

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def batch_of(lay, per_group_ids, budget):
    slots = np.concatenate([np.asarray(x, np.int64) for x in per_group_ids]) if per_group_ids else np.zeros(0, np.int64)
    off = np.concatenate([[0], np.cumsum([len(x) for x in per_group_ids])]).astype(np.int64)
    return workloads.SlotBatch(lay, slots, off, off, budget)


@pytest.mark.parametrize("flags", [0, capi.RT_PLAN_TMA], ids=["ld128", "tma"])
@pytest.mark.parametrize("dtype", [np.int64, np.int32], ids=["i64", "i32"])
def test_state_after_capacity_and_slot_range_errors(flags, dtype):
    if flags and dtype == np.int32:
        pytest.skip("the bulk-copy kernel reads int64 ids")
    lay = workloads.Layout(3, 2048, 65536, shared_bitmap=False)          # 3 bitmaps x 64 blocks, 6 buffers
    T = lay.block_tokens
    before = [{1, 2, 3, 40}, {5}, set()]
    # every second block: 16 runs per buffer and phase -- far more than 24 ranges
    spread = batch_of(lay, [np.arange(0, 32, 2) * T + 7] * 3, 64)
    bad = batch_of(lay, [[9, 10, lay.capacity + 1, 1 << 40], [3 * T + 1], [5]], 8)
    good = batch_of(lay, [[2 * T + 1, 9 * T + 5], [5 * T + 2, 6 * T], [T + 1]], 8)
    p = DevicePlanner(lay, 0, max_indices=256, max_ranges=24)
    p.set_resident(before)
    f = flags | capi.RT_PLAN_EVICT

    with pytest.raises(capi.RtError) as e:
        p.step_host(spread.slots.astype(dtype), spread.group_off, spread.budget_blocks, f)
    assert e.value.status == capi.RT_ERR_CAPACITY
    assert p.get_resident() == [sorted(s) for s in before]

    with pytest.raises(capi.RtError) as e:
        p.step_host(bad.slots.astype(dtype) if dtype == np.int64 else
                    np.where(bad.slots > 2**31 - 1, 2**31 - 1, bad.slots).astype(dtype),
                    bad.group_off, bad.budget_blocks, f)
    assert e.value.status == capi.RT_ERR_SLOT_RANGE
    assert p.get_resident() == [sorted(s) for s in before]

    # the next valid step plans from the untouched state, exactly like the oracle
    resident = [set(s) for s in before]
    want, info = compose.plan_step(good, resident, evict=True)
    got, res = p.step_host(good.slots.astype(dtype), good.group_off, good.budget_blocks, f)
    assert ranges_to_tuples(got) == want and res.flags == 0
    assert res.blocks_evicted == info["blocks_evicted"] > 0
    assert p.get_resident() == [sorted(s) for s in resident]
    p.close()


def test_device_side_overflow_reports_the_need_and_commits_nothing():
    lay = workloads.Layout(2, 2048, 65536, shared_bitmap=True)
    T = lay.block_tokens
    dev = torch.device("cuda:0")
    ids = torch.from_numpy(np.arange(0, 40, 2, dtype=np.int64) * T + 3).to(dev)      # 20 runs x 4 buffers
    off = np.array([0, ids.numel()], np.int64)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    small = torch.zeros(8 * 24, dtype=torch.uint8, device=dev)
    big = torch.zeros(256 * 24, dtype=torch.uint8, device=dev)
    p = DevicePlanner(lay, 0)
    p.set_resident([{63}])
    p.step_device(ids, off, 64, capi.RT_PLAN_EVICT, small, d_res)
    p.sync()
    r = result_from_tensor(d_res)
    assert r["flags"] == capi.RT_RESULT_OVERFLOW and r["n_ranges"] == 4 * 20 + 4
    assert p.get_resident() == [[63]]
    p.step_device(ids, off, 64, capi.RT_PLAN_EVICT, big, d_res)
    p.sync()
    r = result_from_tensor(d_res)
    assert r["flags"] == 0 and r["n_ranges"] == 84 and r["n_cpu_ranges"] == 4
    assert p.get_resident() == [list(range(0, 40, 2))]
    # bitmaps given, no scan: same rule
    p.set_resident([{63}])
    want = torch.zeros(32, dtype=torch.int32, device=dev)
    want[0] = 0x55555555
    p.from_bitmaps(want, 64, capi.RT_PLAN_EVICT, small, d_res)
    p.sync()
    assert result_from_tensor(d_res)["flags"] == capi.RT_RESULT_OVERFLOW and p.get_resident() == [[63]]
    p.close()


@pytest.mark.parametrize("shared", [True, False])
def test_a_bitmap_that_moves_nothing_keeps_its_record(shared):
    """Without eviction: blocks that are committed but not desired right now stay on
    record as long as nothing is sent for that bitmap, and are not sent again
    when they return."""
    lay = workloads.Layout(2, 2048, 65536, shared_bitmap=shared)
    T = lay.block_tokens
    G = lay.n_groups
    steps = [batch_of(lay, [[T + 1, 2 * T + 1, 3 * T + 1]] * G, 8),
             batch_of(lay, [[2 * T + 9]] * G, 8),                     # a subset: nothing to send
             batch_of(lay, [[T + 1, 2 * T + 1, 3 * T + 1]] * G, 8),   # they are still on record
             batch_of(lay, [[2 * T + 9, 7 * T]] * G, 8),              # something is sent: the record shrinks
             batch_of(lay, [[T + 5]] * G, 8)]                         # ... so block 1 goes out again
    p = DevicePlanner(lay, 0, max_indices=64)
    resident = [set() for _ in range(G)]
    sent = []
    for b in steps:
        want, _ = compose.plan_step(b, resident, evict=False)
        got, res = p.step_host(b.slots, b.group_off, b.budget_blocks, 0)
        assert ranges_to_tuples(got) == want
        assert p.get_resident() == [sorted(s) for s in resident]
        sent.append(res.blocks_added // G)
    assert sent == [3, 0, 0, 1, 1]
    assert p.get_resident() == [[1]] * G           # what was still desired, plus what was sent
    p.close()


def test_feedback_plan_overflow_commits_nothing():
    """rt_feedback_plan with a range buffer that is too small: neither the
    resident words nor the per-block commit stamps change, so the same plan
    comes out in full once the buffer is large enough."""
    lay = workloads.Layout(4, 2048, 65536, shared_bitmap=True)
    T = lay.block_tokens
    dev = torch.device("cuda:0")
    spec = rp.SlotSpec(block_tokens=T, max_blocks_per_update=16, active_seconds=2.0, refresh_seconds=10.0)
    oracle = compose.FeedbackSession(lay, spec, 16, evict=True)
    planner = DevicePlanner(lay, 0)
    fb = DeviceFeedback(planner, pid=0)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    small = torch.zeros(4 * 24, dtype=torch.uint8, device=dev)
    big = torch.zeros(1024 * 24, dtype=torch.uint8, device=dev)
    kw = dict(budget=16, max_blocks_per_update=16, active_seconds=2.0, refresh_seconds=10.0,
              flags=capi.RT_PLAN_EVICT, d_result=d_res)
    reads = np.arange(0, 24, 2, dtype=np.int64) * T + 1                 # 12 separate blocks
    alloc = np.arange(1, 50, dtype=np.int64)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    fb.alloc(up(alloc), 100.0, None)
    oracle.alloc(alloc, None, 100.0)
    fb.attention(up(reads), up(np.zeros(0, np.int64)), 100.1)
    oracle.attention(reads, np.zeros(0, np.int64), 100.1)
    fb.plan(100.2, d_out=small, **kw)
    torch.cuda.synchronize()
    r = result_from_tensor(d_res)
    assert r["flags"] == capi.RT_RESULT_OVERFLOW and r["n_ranges"] > 4
    assert planner.get_resident() == [[]]
    fb.plan(100.3, d_out=big, **kw)
    want, info = oracle.plan(100.3)
    torch.cuda.synchronize()
    r = result_from_tensor(d_res)
    assert r["flags"] == 0
    assert ranges_to_tuples(ranges_from_tensor(big, r["n_ranges"])) == want and len(want) > 4
    assert planner.get_resident()[0] == info["committed"]
    # nothing is due a moment later: the commit stamps were written by the second plan only
    fb.plan(100.4, d_out=big, **kw)
    want, _ = oracle.plan(100.4)
    torch.cuda.synchronize()
    assert want == [] and result_from_tensor(d_res)["n_ranges"] == 0
    fb.close()
    planner.close()
