"""GPU parity of the device-resident entry points over seeded random geometries:
ids already in HBM (one flat list with per-bitmap offsets), the padded request
table with a random stride, and the scan-only call followed by the plan from
bitmaps (plus, for 64-bit ids, the allocation-free scan).  All three must give
the CPU oracle's range list from the same random resident set, for 64- and
32-bit ids; the scans' bitmaps must equal the set of blocks the oracle finds,
bit for bit."""
import ctypes as C
import dataclasses
import os

import numpy as np
import pytest

from oracle import compose
from retarget_b200 import capi
from retarget_b200.planner import (DevicePlanner, blocks_to_bitmap, ranges_from_tensor,
                                   ranges_to_tuples, result_from_tensor)
from test_gpu_plan_fuzz import random_shape
from test_gpu_plan_parity import random_batch

pytestmark = pytest.mark.gpu

# RETARGET_FUZZ_SEEDS=N runs a longer sweep of the same generator
SEEDS = int(os.environ.get("RETARGET_FUZZ_SEEDS", 16))
torch = pytest.importorskip("torch")


@pytest.mark.parametrize("dtype", [np.int64, np.int32], ids=["i64", "i32"])
@pytest.mark.parametrize("seed", range(SEEDS))
def test_device_entry_points(seed, dtype):
    rng = np.random.default_rng(5200 + seed)
    shape = random_shape(rng)
    b = random_batch(rng, **shape)
    b = dataclasses.replace(b, slots=b.slots.astype(dtype))
    lay = b.layout
    G = lay.n_groups
    evict = bool(seed & 1)
    flags = capi.RT_PLAN_EVICT if evict else 0
    # a random resident set within the budget, so that the plan both adds and evicts
    resident0 = [set(rng.choice(lay.n_blocks, min(lay.n_blocks, int(rng.integers(0, b.budget_blocks + 1))),
                                replace=False).tolist()) for _ in range(G)]
    after = [set(s) for s in resident0]
    want, _ = compose.plan_step(b, after, evict=evict)

    dev = torch.device("cuda:0")
    d_slots = torch.from_numpy(np.ascontiguousarray(b.slots)).to(dev)
    d_out = torch.zeros((1 << 16) * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    stream = torch.cuda.Stream(device=dev).cuda_stream
    torch.cuda.synchronize()

    def fresh():
        p = DevicePlanner(lay, 0, max_indices=0, max_ranges=1 << 16)
        p.set_resident(resident0)
        return p

    def check(p, what):
        torch.cuda.synchronize()
        res = result_from_tensor(d_res)
        assert ranges_to_tuples(ranges_from_tensor(d_out, res["n_ranges"])) == want, what
        assert [sorted(s) for s in after] == p.get_resident(), what
        p.close()

    p = fresh()
    p.step_device(d_slots, b.group_off, b.budget_blocks, flags, d_out, d_res, stream)
    check(p, "ids in HBM")

    p = fresh()
    d_bits = torch.zeros(G * capi.RT_BITMAP_WORDS, dtype=torch.int32, device=dev)
    p.scan(d_slots, b.group_off, d_bits, d_res, stream)
    torch.cuda.synchronize()
    bits = d_bits.cpu().numpy().view(np.uint32).reshape(G, capi.RT_BITMAP_WORDS)
    touched = 0
    for g in range(G):
        blocks = compose.touched_blocks(b.slots[b.group_off[g]:b.group_off[g + 1]], lay)
        assert np.array_equal(bits[g], blocks_to_bitmap(blocks)), g
        touched += len(blocks)
    assert result_from_tensor(d_res)["blocks_touched"] == touched
    p.from_bitmaps(d_bits, b.budget_blocks, flags, d_out, d_res, stream)
    check(p, "scan, then plan from bitmaps")

    if dtype is np.int64:      # the allocation-free scan takes 64-bit ids
        d_static = torch.full((G * capi.RT_BITMAP_WORDS,), -1, dtype=torch.int32, device=dev)
        fn = capi.lib.rt_scan_slots_static
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint32, C.c_uint32,
                       C.c_void_p, C.c_void_p, C.c_void_p]
        status = fn(d_slots.data_ptr() if d_slots.numel() else None, b.group_off.ctypes.data, G, lay.capacity,
                    lay.block_tokens, lay.n_blocks, d_static.data_ptr(), d_res.data_ptr(), stream)
        assert status == 0, capi.strerror(status)
        torch.cuda.synchronize()
        assert np.array_equal(d_static.cpu().numpy().view(np.uint32).reshape(G, -1), bits)
        assert result_from_tensor(d_res)["blocks_touched"] == touched

    if G == 1:      # the request table feeds one bitmap
        lens = np.diff(b.req_off).astype(np.int32)
        stride = int(lens.max()) + int(rng.integers(0, 9))
        if stride:
            table = np.full((len(lens), stride), -7, dtype=dtype)
            for r, n in enumerate(lens):
                table[r, :n] = b.slots[b.req_off[r]:b.req_off[r + 1]]
            p = fresh()
            p.step_table(torch.from_numpy(table).to(dev), torch.from_numpy(lens).to(dev), b.budget_blocks,
                         flags, d_out, d_res, stream)
            check(p, "request table")
