"""The host-buffer call narrows large lists of 64-bit ids to 32 bits before the
copy.  Its plan, its counters and the state it leaves must be those of the call
that copies the ids as they are, and the oracle's."""
import numpy as np
import pytest

from oracle import compose
from retarget_b200 import capi, workloads
from retarget_b200.planner import DevicePlanner, ranges_to_tuples

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(autouse=True)
def narrowing_on(monkeypatch):
    """Narrow whatever the host looks like (the default rule wants 8 threads per GPU)."""
    monkeypatch.setenv("RETARGET_B200_PACK_THREADS", "6")


def both(layout, slots, group_off, budget, flags, **kw):
    out = []
    for extra in (0, capi.RT_PLAN_WIDE_COPY):
        p = DevicePlanner(layout, 0, max_indices=len(slots) + 8)
        got, res = p.step_host(slots, group_off, budget, flags | extra, **kw)
        out.append((ranges_to_tuples(got), res.as_dict(), p.get_resident()))
        p.close()
    return out


@pytest.mark.parametrize("lead", [0, 1, 3], ids=["aligned", "lead1", "lead3"])
def test_narrowed_call_matches_wide_call_and_oracle(lead):
    """11.1 M ids (above the 2^20 threshold, not a multiple of the chunk), read from
    pageable memory at three alignments."""
    b = workloads.sparse_feedback(lead)
    padded = np.concatenate([np.zeros(lead, np.int64), b.slots])
    slots = padded[lead:]
    assert len(slots) >= 1 << 20 and len(slots) % (1 << 21)
    narrow, wide = both(b.layout, slots, b.group_off, b.budget_blocks, capi.RT_PLAN_EVICT)
    assert narrow == wide
    want, info = compose.plan_step(b, [set() for _ in range(b.layout.n_groups)], evict=True)
    assert narrow[0] == want and narrow[1]["blocks_added"] == info["blocks_added"]


def test_ids_outside_32_bits_keep_their_class():
    """Negative ids (ignored), ids above the capacity and ids that do not fit 32
    bits (out of range) are counted the same by both calls; nothing is committed."""
    b = workloads.sparse_feedback(7, layers=8)
    slots = b.slots.copy()
    assert len(slots) >= 1 << 20
    rng = np.random.default_rng(3)
    at = rng.choice(len(slots), size=40, replace=False)
    bad = np.array([-1, -2**31, -2**31 - 1, -2**40, np.iinfo(np.int64).min, 0, 0, 0], dtype=np.int64)
    big = np.array([b.layout.capacity + 1, 2**31 - 1, 2**31, 2**32, 2**32 + 5, 2**40, np.iinfo(np.int64).max],
                   dtype=np.int64)
    slots[at[:len(bad)]] = bad
    narrow, wide = both(b.layout, slots, b.group_off, b.budget_blocks, capi.RT_PLAN_EVICT, raise_on_slot_range=False)
    assert narrow == wide
    assert narrow[1]["ignored_slots"] >= len(bad) and narrow[1]["invalid_slots"] == 0
    slots[at[20:20 + len(big)]] = big
    narrow, wide = both(b.layout, slots, b.group_off, b.budget_blocks, capi.RT_PLAN_EVICT, raise_on_slot_range=False)
    assert narrow == wide
    assert narrow[1]["invalid_slots"] == len(big) and narrow[1]["flags"] & capi.RT_RESULT_SLOT_RANGE
    assert narrow[2] == [[] for _ in range(b.layout.n_groups)]


def test_thread_rule(monkeypatch):
    lay = workloads.Layout(1, 2048, 8192)
    for text, want in (("0", 0), ("1", 1), ("12", 12), ("500", 64)):
        monkeypatch.setenv("RETARGET_B200_PACK_THREADS", text)
        p = DevicePlanner(lay, 0, max_indices=64)
        assert p.narrow_threads() == want
        p.close()
    monkeypatch.delenv("RETARGET_B200_PACK_THREADS")
    p = DevicePlanner(lay, 0, max_indices=64)
    assert p.narrow_threads() == 0 or 8 <= p.narrow_threads() <= 16
    if torch.cuda.device_count() > 1:
        assert p.narrow_threads() == 0          # several GPUs visible: the planners share the host
    p.close()


def test_chained_host_steps_keep_state():
    """Three host-buffer steps in a row through the narrowed path follow the oracle's
    resident sets (the staging buffer is reused from call to call)."""
    a, b = workloads.target_pair("moving")
    p = DevicePlanner(a.layout, 0, max_indices=a.n_idx + 8)
    resident = [set() for _ in range(a.layout.n_groups)]
    for batch in (a, b, a):
        want, _ = compose.plan_step(batch, resident, evict=True)
        got, res = p.step_host(batch.slots, batch.group_off, batch.budget_blocks, capi.RT_PLAN_EVICT)
        assert ranges_to_tuples(got) == want
    p.close()
