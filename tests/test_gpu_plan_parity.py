"""GPU parity: the CUDA planner, called through the C ABI, against the CPU
oracle on the same seeded inputs.  Integer work: every comparison is exact."""
import dataclasses

import numpy as np
import pytest

from oracle import compose
from oracle import ref_policy as rp
from oracle import uvm_expand as ux
from retarget_b200 import capi, workloads
from retarget_b200.planner import (DevicePlanner, blocks_to_bitmap, ranges_from_tensor,
                                   ranges_to_tuples, result_from_tensor)

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

# (flags, id dtype): the register-staged kernel, the bulk-copy kernel, and the
# register-staged kernel reading 32-bit ids
MODES = [pytest.param((0, np.int64), id="ld128"), pytest.param((capi.RT_PLAN_TMA, np.int64), id="tma"),
         pytest.param((0, np.int32), id="i32")]


def random_batch(rng, *, layers, pool_slots, bytes_per_slot, shared, n_req, max_len, budget,
                 block_bytes=2 << 20, junk=False):
    lay = workloads.Layout(layers, bytes_per_slot, pool_slots, block_bytes, shared)
    G = lay.n_groups
    chunks, lens = [], []
    for g in range(G):
        for r in range(n_req):
            n = int(rng.integers(0, max_len + 1))
            kind = rng.integers(0, 3)
            if kind == 0:      # paged, consecutive within a page
                pages = rng.integers(0, max(1, pool_slots // 16), -(-n // 16))
                s = (pages[:, None] * 16 + np.arange(16)).reshape(-1)[:n]
            elif kind == 1:    # one long consecutive run
                start = int(rng.integers(0, max(1, pool_slots - n)))
                s = np.arange(start, start + n)
            else:              # random with repeats
                s = rng.integers(1, pool_slots, n)
            s = np.clip(s, 0, lay.capacity).astype(np.int64)
            if junk and n:
                k = rng.integers(0, n, max(1, n // 50))
                s[k] = rng.choice([0, -1, -5, -(1 << 40)], len(k))
            chunks.append(s)
            lens.append(n)
    slots = np.concatenate(chunks) if chunks else np.zeros(0, np.int64)
    req_off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    group_off = req_off[::n_req].copy() if n_req else np.zeros(G + 1, np.int64)
    return workloads.SlotBatch(lay, slots.astype(np.int64), group_off, req_off, budget, "random")


class CChain:
    """The literal chain in C (oracle/plan_oracle.c: encode_runs -> blocks ->
    one-event ranking -> choose -> blocksv run walk), for inputs on which the
    Python restatement would take minutes."""

    def __init__(self, layout):
        from oracle import c_oracle
        self.c = c_oracle.COracle(layout)

    def step(self, b, evict):
        before = self.c.resident_sets()
        out, invalid = self.c.step(np.ascontiguousarray(b.slots, dtype=np.int64), b.group_off, b.budget_blocks, evict)
        assert invalid == 0
        after = self.c.resident_sets()
        info = dict(blocks_added=sum(len(x - y) for x, y in zip(after, before)),
                    blocks_evicted=sum(len(y - x) for x, y in zip(after, before)) if evict else 0)
        return ranges_to_tuples(out), info, after


def run_steps(batches, *, evict, flags, literal=True):
    """Feeds the same sequence of batches to the device planner (host-buffer
    entry point) and to the oracle; compares every step.  ``literal=True``: the
    Python restatement of the reference chain; ``literal=False``: the same chain
    in C (sizes the Python loops cannot finish in seconds)."""
    flags, dtype = flags if isinstance(flags, tuple) else (flags, np.int64)
    lay = batches[0].layout
    planner = DevicePlanner(lay, 0, max_indices=max(b.n_idx for b in batches) + 8, max_ranges=1 << 16)
    resident = [set() for _ in range(lay.n_groups)]
    chain = None if literal else CChain(lay)
    f = flags | (capi.RT_PLAN_EVICT if evict else 0)
    for step, b in enumerate(batches):
        # oracle and planner both see the ids in the dtype under test
        b = dataclasses.replace(b, slots=b.slots.astype(dtype))
        if literal:
            want, info = compose.plan_step(b, resident, evict=evict, literal=True)
        else:
            want, info, resident = chain.step(b, evict)
        got, res = planner.step_host(b.slots, b.group_off, b.budget_blocks, f)
        assert ranges_to_tuples(got) == want, f"step {step}"
        assert res.n_ranges == len(want)
        assert res.n_cpu_ranges == sum(1 for r in want if r[1] == ux.CPU)
        assert res.blocks_added == info["blocks_added"]
        assert res.blocks_evicted == info["blocks_evicted"]
        assert res.gpu_bytes == sum(r[3] for r in want if r[1] != ux.CPU)
        assert res.cpu_bytes == sum(r[3] for r in want if r[1] == ux.CPU)
        assert res.invalid_slots == 0
        assert [sorted(s) for s in resident] == planner.get_resident(), f"step {step}"
    planner.close()


@pytest.mark.parametrize("flags", MODES)
@pytest.mark.parametrize("evict", [True, False])
def test_random_small_multi_step(flags, evict):
    rng = np.random.default_rng(42)
    shapes = [
        dict(layers=3, pool_slots=8192, bytes_per_slot=2048, shared=False, n_req=5, max_len=700, budget=3),
        dict(layers=2, pool_slots=65536, bytes_per_slot=2048, shared=True, n_req=9, max_len=5000, budget=16),
        dict(layers=4, pool_slots=262144, bytes_per_slot=256, shared=False, n_req=3, max_len=9000, budget=8),
        # 1024 blocks of 4 KiB: the widest bitmap the protocol allows
        dict(layers=2, pool_slots=8192, bytes_per_slot=512, shared=False, n_req=6, max_len=3000,
             budget=300, block_bytes=4096),
        # 6 slots per block (not a power of two), 1001 blocks, the last one partial
        dict(layers=2, pool_slots=6001, bytes_per_slot=2048, shared=False, n_req=4, max_len=2500,
             budget=40, block_bytes=12288),
    ]
    for shape in shapes:
        batches = [random_batch(rng, junk=(k == 2), **shape) for k in range(4)]
        # vary the budget between steps as a scheduler would
        batches[3] = dataclasses.replace(batches[3], budget_blocks=max(1, shape["budget"] // 2))
        run_steps(batches, evict=evict, flags=flags)


@pytest.mark.parametrize("evict", [True, False])
def test_wide_layouts(evict):
    """Shapes that take the tail's general paths: more bitmaps than one pass of
    the CTA holds (100 x 1024 blocks), more (phase, buffer) pairs than threads
    (200 and 300 buffers), long run lists, a partial last block."""
    rng = np.random.default_rng(11)
    shapes = [
        # 100 bitmaps of 1024 blocks, 200 buffers
        dict(layers=100, pool_slots=8192, bytes_per_slot=512, shared=False, n_req=2, max_len=1500,
             budget=200, block_bytes=4096),
        # one bitmap shared by 300 buffers, 1001 blocks of 6 slots, last block partial
        dict(layers=150, pool_slots=6001, bytes_per_slot=2048, shared=True, n_req=5, max_len=2500,
             budget=80, block_bytes=12288),
        # 128 bitmaps (the most a plan can hold), 256 buffers, 64 blocks
        dict(layers=128, pool_slots=65536, bytes_per_slot=2048, shared=False, n_req=2, max_len=3000,
             budget=9),
    ]
    for shape in shapes:
        batches = [random_batch(rng, **shape) for _ in range(3)]
        batches.append(dataclasses.replace(batches[0], budget_blocks=max(1, shape["budget"] // 3)))
        run_steps(batches, evict=evict, flags=(0, np.int64), literal=False)


@pytest.mark.parametrize("flags", MODES)
def test_ragged_and_empty_inputs(flags):
    rng = np.random.default_rng(7)
    lay = workloads.Layout(4, 2048, 32768, shared_bitmap=False)
    # groups: empty, one id at an odd offset, a few ids, empty
    slots = np.array([77, 5000, 5001, 5002, 31000, 1, 1], dtype=np.int64)
    b0 = workloads.SlotBatch(lay, slots, np.array([0, 0, 1, 7, 7], np.int64),
                             np.array([0, 0, 1, 7, 7], np.int64), 2)
    empty = workloads.SlotBatch(lay, np.zeros(0, np.int64), np.zeros(5, np.int64),
                                np.zeros(5, np.int64), 2)
    zero_budget = dataclasses.replace(b0, budget_blocks=0)
    big = random_batch(rng, layers=4, pool_slots=32768, bytes_per_slot=2048, shared=False,
                       n_req=3, max_len=4099, budget=50)
    run_steps([b0, empty, b0, zero_budget, big, empty], evict=True, flags=flags)


@pytest.mark.parametrize("flags", MODES)
def test_full_refresh_config(flags):
    """40 layers, 65,536-slot pool, 64 requests, 25 % budget: literal oracle."""
    b = workloads.full_refresh(0)
    assert b.layout.n_blocks == 64 and b.budget_blocks == 16 and b.layout.n_buffers == 80
    b2 = workloads.full_refresh(1)
    run_steps([b, b, b2], evict=True, flags=flags)


@pytest.mark.parametrize("flags", MODES)
def test_tp_shard_config(flags):
    """48 layers, one KV head per rank (256 B slots), 262,144-slot pool."""
    b = workloads.tp_shard(0)
    assert b.layout.n_blocks == 32 and b.layout.block_tokens == 8192 and b.layout.n_buffers == 96
    run_steps([b, workloads.tp_shard(3)], evict=True, flags=flags, literal=False)


def test_sparse_feedback_config_reduced_literal():
    """Per-layer touched sets (newest 128 + 2048 Zipf draws), 4 layers through
    the literal reference chain."""
    b = workloads.sparse_feedback(0, layers=4, requests=32)
    assert b.layout.n_groups == 4 and b.layout.n_blocks == 128 and b.budget_blocks == 19
    run_steps([b, workloads.sparse_feedback(1, layers=4, requests=32)], evict=True, flags=0)


@pytest.mark.parametrize("flags", MODES)
def test_sparse_feedback_config_full(flags):
    """Full 40-layer, 128-request case (11.1 M ids)."""
    b = workloads.sparse_feedback(0)
    assert b.n_idx == 128 * 40 * 2176
    run_steps([b, b], evict=True, flags=flags, literal=False)


@pytest.mark.parametrize("dtype", [np.int64, np.int32], ids=["i64", "i32"])
def test_device_resident_entry_points_agree(dtype):
    """step_device (ids already in HBM), the padded-table entry point and the
    scan-only + from-bitmaps pair all give the host-buffer call's answer."""
    b = workloads.full_refresh(2)
    b = dataclasses.replace(b, slots=b.slots.astype(dtype))
    lay = b.layout
    dev = torch.device("cuda:0")
    resident0 = [set(range(3, 9))]
    want, _ = compose.plan_step(b, [set(resident0[0])], evict=True)
    d_slots = torch.from_numpy(b.slots).to(dev)
    d_out = torch.zeros(4096 * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    side = torch.cuda.Stream(device=dev)        # the caller's own stream
    stream = side.cuda_stream
    torch.cuda.synchronize()

    def fresh():
        p = DevicePlanner(lay, 0, max_indices=0)
        p.set_resident(resident0)
        return p

    p = fresh()
    p.step_device(d_slots, b.group_off, b.budget_blocks, capi.RT_PLAN_EVICT, d_out, d_res, stream)
    torch.cuda.synchronize()
    res = result_from_tensor(d_res)
    assert ranges_to_tuples(ranges_from_tensor(d_out, res["n_ranges"])) == want
    p.close()

    # padded [requests, stride] table with an odd stride
    lens = np.diff(b.req_off).astype(np.int32)
    stride = int(lens.max()) + 3
    table = np.full((len(lens), stride), -7, dtype=dtype)
    for r, n in enumerate(lens):
        table[r, :n] = b.slots[b.req_off[r]:b.req_off[r + 1]]
    p = fresh()
    p.step_table(torch.from_numpy(table).to(dev), torch.from_numpy(lens).to(dev), b.budget_blocks,
                 capi.RT_PLAN_EVICT, d_out, d_res, stream)
    torch.cuda.synchronize()
    res = result_from_tensor(d_res)
    assert ranges_to_tuples(ranges_from_tensor(d_out, res["n_ranges"])) == want
    assert res["ignored_slots"] == 0          # padding is never read
    p.close()

    # scan only, then diff + coalesce from the bitmap
    p = fresh()
    d_bits = torch.zeros(32, dtype=torch.int32, device=dev)
    p.scan(d_slots, b.group_off, d_bits, d_res, stream)
    torch.cuda.synchronize()
    touched = compose.touched_blocks(b.slots, lay)
    assert np.array_equal(d_bits.cpu().numpy().view(np.uint32), blocks_to_bitmap(touched))
    assert result_from_tensor(d_res)["blocks_touched"] == len(touched)
    p.from_bitmaps(d_bits, b.budget_blocks, capi.RT_PLAN_EVICT, d_out, d_res, stream)
    torch.cuda.synchronize()
    res = result_from_tensor(d_res)
    assert ranges_to_tuples(ranges_from_tensor(d_out, res["n_ranges"])) == want
    p.close()


def test_window_plan_from_bitmaps_matches_window_command():
    """A block-aligned window held as a bitmap: resident = old window, wanted =
    new window gives exactly the windowv symmetric difference."""
    lay = workloads.Layout(40, 2048, 65536)
    spec = rp.WindowSpec(lay.alloc_bytes, lay.n_buffers, 2048, 16384, 8192, 1024)
    dev = torch.device("cuda:0")
    d_out = torch.zeros(4096 * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    p = DevicePlanner(lay, 0)
    old = None
    for completed in (100, 9000, 9100, 30000, 12, 1 << 30):
        new, want = compose.window_step(spec, lay, completed, old)
        if old is None:
            # first plan: everything outside the window to the CPU, window to the GPU
            p.set_resident([set(range(lay.n_blocks))])
        want_bits = torch.from_numpy(
            blocks_to_bitmap(compose.window_blocks(*new, lay.block_bytes)).view(np.int32)).to(dev)
        p.from_bitmaps(want_bits, capi.RT_MAX_BLOCKS, capi.RT_PLAN_EVICT, d_out, d_res)
        p.sync()
        res = result_from_tensor(d_res)
        got = ranges_to_tuples(ranges_from_tensor(d_out, res["n_ranges"]))
        if old is None:
            # the command also re-sends the window itself; the bitmap diff only moves what changes
            want = [r for r in want if r[1] == ux.CPU]
        assert got == want, completed
        old = new
    p.close()


def test_slot_above_capacity_is_reported():
    lay = workloads.Layout(2, 2048, 8192)
    slots = np.array([5, 8191, 8192, 1 << 40, 9], dtype=np.int64)
    p = DevicePlanner(lay, 0, max_indices=16)
    with pytest.raises(capi.RtError) as e:
        p.step_host(slots, np.array([0, 5], np.int64), 4)
    assert e.value.status == capi.RT_ERR_SLOT_RANGE
    got, res = p.step_host(slots, np.array([0, 5], np.int64), 4, raise_on_slot_range=False)
    assert res.invalid_slots == 2 and res.flags & capi.RT_RESULT_SLOT_RANGE
    # counters are clean again on the next step
    got, res = p.step_host(slots[:2], np.array([0, 2], np.int64), 4)
    assert res.invalid_slots == 0 and res.flags == 0
    p.close()


@pytest.mark.parametrize("shared", [True, False])
def test_partial_last_block_is_clamped(shared):
    """Plans that include the final, partial block of every buffer: its range
    ends at the allocation size (select.cpp:24188) and the byte totals count it
    short, when it is added and when it is evicted again."""
    lay = workloads.Layout(3, 2048, 6001, 12288, shared)          # 1001 blocks of 6 slots, 1 slot in the last
    assert lay.n_blocks == 1001 and lay.alloc_bytes % lay.block_bytes == 2048
    G = lay.n_groups
    tail_ids = np.array([5990, 5995, 6000, 5999, 17], dtype=np.int64)     # blocks 998, 999, 1000, 2
    head_ids = np.array([1, 7, 13], dtype=np.int64)
    def batch(ids, budget):
        slots = np.tile(ids, G)
        off = np.arange(G + 1, dtype=np.int64) * len(ids)
        return workloads.SlotBatch(lay, slots, off, off, budget)
    steps = [batch(tail_ids, 10), batch(head_ids, 10), batch(tail_ids, 3), batch(tail_ids, 10)]
    run_steps(steps, evict=True, flags=(0, np.int64))
    # the figure itself, once: 4 blocks per buffer, the last one 2048 bytes long
    p = DevicePlanner(lay, 0, max_indices=64)
    got, res = p.step_host(steps[0].slots, steps[0].group_off, 10, capi.RT_PLAN_EVICT)
    assert res.gpu_bytes == lay.n_buffers * (3 * 12288 + 2048)
    assert int(got["offset"].max() + got["bytes"][got["offset"].argmax()]) == lay.alloc_bytes
    p.close()


@pytest.mark.parametrize("flags", MODES)
def test_reference_qwen_geometry(flags):
    """The reference's own deployment: 80 KV allocations of 448,790,528 bytes
    (219,136 slots of 2048 bytes), 256-token blocks (856 of 512 KiB), one mask for all allocations, a 32,768-token budget
    (128 blocks).  Python chain on the first two steps, the same chain in C after."""
    rng = np.random.default_rng(23)
    shape = dict(layers=40, pool_slots=219136, bytes_per_slot=2048, shared=True, n_req=24, max_len=4096,
                 budget=32768 // 256, block_bytes=256 * 2048)
    batches = [random_batch(rng, **shape) for _ in range(4)]
    lay = batches[0].layout
    assert lay.alloc_bytes == 448790528 and lay.n_buffers == 80 and lay.n_blocks == 856
    run_steps(batches[:2], evict=True, flags=flags, literal=True)
    run_steps(batches, evict=True, flags=flags, literal=False)
    run_steps(batches, evict=False, flags=flags, literal=False)


@pytest.mark.parametrize("kind", ["moving", "fragmented"])
def test_benchmark_pairs_match_oracle(kind):
    """The alternating batches the benchmark times: every step evicts and adds
    (160 ranges when the halves alternate, 6080 single-block ranges when even
    and odd blocks do)."""
    a, b = workloads.target_pair(kind)
    run_steps([a, b, a], evict=True, flags=(0, np.int64), literal=False)
    want = {"moving": 160, "fragmented": 6080}[kind]
    chain = CChain(a.layout)
    chain.step(a, True)
    ranges, _, _ = chain.step(b, True)
    assert len(ranges) == want


def test_int32_ids_negative_and_above_capacity():
    """32-bit ids: negatives are ignored like any id below 1, ids above the
    capacity are counted, and an odd start offset inside a 16-byte vector works."""
    lay = workloads.Layout(2, 2048, 8192)
    slots = np.array([99, 5, -3, 8191, 8192, 2**31 - 1, 9, -2**31, 0, 4000, 4001], dtype=np.int32)
    p = DevicePlanner(lay, 0, max_indices=64)
    # ids [1, 11): starts at index 1 of the first 4-id vector
    got, res = p.step_host(slots, np.array([1, 11], np.int64), 8, raise_on_slot_range=False)
    assert res.invalid_slots == 2 and res.ignored_slots == 3
    assert res.flags & capi.RT_RESULT_SLOT_RANGE
    assert p.get_resident() == [[]]              # a step that failed commits nothing
    # the same ids without the two that are out of range
    ok = slots[(slots <= lay.capacity)].copy()
    got, res = p.step_host(ok, np.array([1, len(ok)], np.int64), 8)
    assert res.invalid_slots == 0 and res.ignored_slots == 3 and res.flags == 0
    assert p.get_resident() == [[0, 3, 7]]
    p.close()
    # a pool too large for 32-bit ids is refused up front
    big = workloads.Layout(1, 1, (1 << 31) + 2, block_bytes=1 << 22)
    pb = DevicePlanner(big, 0, max_indices=16)
    with pytest.raises(capi.RtError) as e:
        pb.step_host(np.array([1], np.int32), np.array([0, 1], np.int64), 1)
    assert e.value.status == capi.RT_ERR_INVALID_ARGUMENT
    pb.close()


def test_int32_matches_int64_at_headline_size():
    """The benchmark's 22.3 M ids as int32 and as int64 give the same plan."""
    b = workloads.target_step(0)
    p64 = DevicePlanner(b.layout, 0, max_indices=b.n_idx + 8)
    p32 = DevicePlanner(b.layout, 0, max_indices=b.n_idx + 8)
    a, ra = p64.step_host(b.slots, b.group_off, b.budget_blocks, capi.RT_PLAN_EVICT)
    c, rc = p32.step_host(b.slots.astype(np.int32), b.group_off, b.budget_blocks, capi.RT_PLAN_EVICT)
    assert ranges_to_tuples(a) == ranges_to_tuples(c) and len(a) > 0
    assert ra.as_dict() == rc.as_dict()
    assert p64.get_resident() == p32.get_resident()
    p64.close()
    p32.close()


def test_range_capacity_overflow_is_reported():
    lay = workloads.Layout(8, 2048, 65536, shared_bitmap=True)
    # every second block touched: 32 runs x 16 buffers
    slots = (np.arange(0, 64, 2, dtype=np.int64) * 1024 + 5)
    p = DevicePlanner(lay, 0, max_indices=64, max_ranges=100)
    with pytest.raises(capi.RtError) as e:
        p.step_host(slots, np.array([0, len(slots)], np.int64), 64)
    assert e.value.status == capi.RT_ERR_CAPACITY
    p.close()


def test_headline_step_properties():
    """At the benchmark's full size (40 layers x 256 requests, 262,144 slots)
    the answer is checked against the literal chain in C and through
    size-independent properties: idempotence, sorted non-overlapping ranges,
    byte accounting."""
    b = workloads.target_step(0)
    lay = b.layout
    p = DevicePlanner(lay, 0, max_indices=b.n_idx + 8)
    want, _, _ = CChain(lay).step(b, True)
    got, res = p.step_host(b.slots, b.group_off, b.budget_blocks, capi.RT_PLAN_EVICT)
    assert ranges_to_tuples(got) == want
    assert res.gpu_bytes == int(got["bytes"].sum()) and res.cpu_bytes == 0
    for j in range(lay.n_buffers):
        mine = got[got["buffer"] == j]
        ends = mine["offset"] + mine["bytes"]
        assert np.all(mine["offset"][1:] > ends[:-1])        # sorted, coalesced, disjoint
        assert np.all(ends <= lay.alloc_bytes)
        assert mine["bytes"].sum() <= b.budget_blocks * lay.block_bytes
    again, res2 = p.step_host(b.slots, b.group_off, b.budget_blocks, capi.RT_PLAN_EVICT)
    assert len(again) == 0 and res2.blocks_added == 0 and res2.blocks_evicted == 0
    p.close()


def _table_case(rng, rows, stride, dtype, lay, fill):
    """A padded request table and the CSR batch holding the same valid ids."""
    if fill == "full":
        lens = np.full(rows, stride, np.int32)
    elif fill == "ragged":
        lens = rng.integers(0, stride + 1, rows).astype(np.int32)
        lens[rng.integers(0, rows, max(1, rows // 7))] = 0
    else:                                   # mostly padding, as in a request pool with few live rows
        lens = np.zeros(rows, np.int32)
        live = rng.choice(rows, max(1, rows // 20), replace=False)
        lens[live] = rng.integers(1, stride + 1, len(live))
    table = rng.integers(lay.capacity + 5, lay.capacity + 900, (rows, stride)).astype(dtype)   # padding: never read
    flat = []
    for r in range(rows):
        n = int(lens[r])
        if n:
            start = int(rng.integers(1, lay.capacity - n)) if n < lay.capacity - 2 and rng.random() < 0.5 else None
            ids = np.arange(start, start + n) if start else rng.integers(0, lay.capacity + 1, n)
            table[r, :n] = ids
            flat.append(ids.astype(np.int64))
    slots = np.concatenate(flat) if flat else np.zeros(0, np.int64)
    off = np.array([0, len(slots)], np.int64)
    return table, lens, workloads.SlotBatch(lay, slots, off, off, 12)


@pytest.mark.parametrize("dtype", [np.int64, np.int32], ids=["i64", "i32"])
def test_request_table_shapes(dtype):
    """The padded-table entry point over the shapes its work split distinguishes:
    many short rows (one segment each), few long rows (cut into segments), odd
    strides (rows off the 16-byte grid), empty rows, a table that is mostly
    padding, and more rows than one pass of a CTA lists."""
    rng = np.random.default_rng(5)
    lay = workloads.Layout(3, 2048, 65536, shared_bitmap=True)
    dev = torch.device("cuda:0")
    d_out = torch.zeros(4096 * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    shapes = [(10240, 96, "full"), (3000, 217, "ragged"), (7, 40001, "ragged"), (64, 20000, "full"),
              (1, 5, "full"), (5000, 33, "sparse"), (3, 1 << 21, "sparse"), (700_000, 6, "ragged")]
    for rows, stride, fill in shapes:
        table, lens, batch = _table_case(rng, rows, stride, dtype, lay, fill)
        chain = CChain(lay)
        p = DevicePlanner(lay, 0)
        for step in range(2):               # the second step plans against what the first left
            if step:
                table, lens, batch = _table_case(rng, rows, stride, dtype, lay, fill)
            want, info, resident = chain.step(batch, True)
            p.step_table(torch.from_numpy(table).to(dev), torch.from_numpy(lens).to(dev), batch.budget_blocks,
                         capi.RT_PLAN_EVICT, d_out, d_res)
            p.sync()
            res = result_from_tensor(d_res)
            assert res["flags"] == 0 and res["invalid_slots"] == 0, (rows, stride, fill)
            assert res["ignored_slots"] == int((batch.slots < 1).sum())
            assert ranges_to_tuples(ranges_from_tensor(d_out, res["n_ranges"])) == want, (rows, stride, fill, step)
            assert p.get_resident() == [sorted(s) for s in resident]
        p.close()


@pytest.mark.parametrize("flags", MODES)
@pytest.mark.parametrize("launch", ["stream", "graph"])
def test_chained_steps_match_the_oracle(flags, launch):
    """RT_PLAN_CHAINED: steps issued back to back, each allowed to start scanning
    while the one before it is still in its tail.  Every step writes to buffers
    of its own, so all plans can be compared afterwards; small steps (tail longer
    than the scan, so tails queue up), medium ones and empty ones are mixed."""
    flag, dtype = flags
    rng = np.random.default_rng(77)
    shape = dict(layers=6, pool_slots=65536, bytes_per_slot=2048, shared=False, n_req=4, budget=9)
    sizes = [40, 30000, 0, 60, 25000, 50, 0, 20, 70000, 35, 10, 45000]
    batches = [random_batch(rng, max_len=n, **shape) for n in sizes]
    lay = batches[0].layout
    dev = torch.device("cuda:0")
    f = flag | capi.RT_PLAN_EVICT | capi.RT_PLAN_CHAINED
    d_slots = [torch.from_numpy(np.ascontiguousarray(b.slots.astype(dtype))).to(dev) for b in batches]
    d_out = [torch.zeros(1024 * 24, dtype=torch.uint8, device=dev) for _ in batches]
    d_res = [torch.zeros(64, dtype=torch.uint8, device=dev) for _ in batches]
    stream = torch.cuda.Stream(device=dev)
    p = DevicePlanner(lay, 0)
    torch.cuda.synchronize()

    def issue(handle):
        for k, b in enumerate(batches):
            p.step_device(d_slots[k], b.group_off, b.budget_blocks, f, d_out[k], d_res[k], handle)

    rounds = 1
    if launch == "stream":
        issue(stream.cuda_stream)
    else:
        rounds = 3                           # captured once, replayed: the state carries over between replays
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            issue(torch.cuda.current_stream().cuda_stream)   # capture only records: nothing runs yet
    resident = [set() for _ in range(lay.n_groups)]
    for r in range(rounds):
        if launch == "graph":
            graph.replay()
        torch.cuda.synchronize()
        for k, b in enumerate(batches):
            want, info = compose.plan_step(b, resident, evict=True, literal=True)
            res = result_from_tensor(d_res[k])
            assert res["flags"] == 0
            assert ranges_to_tuples(ranges_from_tensor(d_out[k], res["n_ranges"])) == want, (r, k)
            assert res["blocks_added"] == info["blocks_added"] and res["blocks_evicted"] == info["blocks_evicted"]
        assert p.get_resident() == [sorted(s) for s in resident]
    p.close()
