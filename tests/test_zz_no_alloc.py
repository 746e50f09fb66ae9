"""The allocation-free scan entry point, ``rt_scan_slots_static``.

Some callers of this library may not allocate device memory: code running
inside the preload library (its own cudaMalloc would pass through the
allocation hook, be registered as a managed allocation and bump the generation
that plans are checked against), and processes whose device memory is owned
entirely by the serving engine's pool.  For them the scan keeps its working
memory in a static device array.  This test calls that entry point through the
C ABI twice in a row -- the second call finds the array as the first one left
it -- and requires the same bitmaps and counters as the plan-based
``rt_scan_slots`` and as the CPU oracle's restatement of the reference's
encode_runs -> blocks chain (integer work: exact equality).

Collected last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import compose
from retarget_b200 import capi, workloads
from retarget_b200.planner import DevicePlanner, blocks_to_bitmap, result_from_tensor

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def scan_both(batch, dev, stream):
    lay = batch.layout
    capi.lib.rt_scan_slots_static.restype = C.c_int
    capi.lib.rt_scan_slots_static.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint32,
                                              C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]
    d_slots = torch.from_numpy(batch.slots).to(dev)
    G = lay.n_groups
    want_bits = torch.full((G * 32,), -1, dtype=torch.int32, device=dev)
    got_bits = torch.full((G * 32,), -1, dtype=torch.int32, device=dev)
    want_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    got_res = torch.full((64,), 255, dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()
    planner = DevicePlanner(lay, 0)
    planner.scan(d_slots, batch.group_off, want_bits, want_res, stream.cuda_stream)
    status = capi.lib.rt_scan_slots_static(
        d_slots.data_ptr(), batch.group_off.ctypes.data, G, lay.capacity, lay.block_tokens, lay.n_blocks,
        got_bits.data_ptr(), got_res.data_ptr(), stream.cuda_stream)
    assert status == 0, capi.strerror(status)
    torch.cuda.synchronize()
    planner.close()
    return (want_bits.cpu().numpy(), result_from_tensor(want_res),
            got_bits.cpu().numpy(), result_from_tensor(got_res))


def test_static_scan_matches_plan_scan_twice_in_a_row():
    dev = torch.device("cuda:0")
    stream = torch.cuda.Stream(device=dev)
    first = workloads.sparse_feedback(3, layers=6, requests=24)
    # second call: other geometry, ragged groups, ids outside 1..capacity
    lay = workloads.Layout(3, 2048, 6001, 12288, False)
    rng = np.random.default_rng(9)
    slots = rng.integers(-2, lay.capacity + 3, 5001).astype(np.int64)
    second = workloads.SlotBatch(lay, slots, np.array([0, 1, 1, 5001], np.int64),
                                 np.array([0, 1, 1, 5001], np.int64), 4)
    for batch in (first, second, first):
        want_bits, want, got_bits, got = scan_both(batch, dev, stream)
        assert np.array_equal(got_bits, want_bits)
        for key in ("blocks_touched", "invalid_slots", "ignored_slots", "flags"):
            assert got[key] == want[key], key
        assert got["n_ranges"] == 0
        # ... and against the oracle itself, bitmap by bitmap
        lay, bits = batch.layout, got_bits.view(np.uint32).reshape(batch.layout.n_groups, 32)
        touched = 0
        for g in range(lay.n_groups):
            ids = batch.slots[batch.group_off[g]:batch.group_off[g + 1]]
            blocks = compose.touched_blocks(ids[ids <= lay.capacity], lay)
            assert np.array_equal(bits[g], blocks_to_bitmap(blocks)), g
            touched += len(blocks)
        assert got["blocks_touched"] == touched
        assert got["invalid_slots"] == int((batch.slots > lay.capacity).sum())
        assert got["ignored_slots"] == int((batch.slots < 1).sum())
    assert want["invalid_slots"] == 0 and want["blocks_touched"] > 0


def test_static_scan_refuses_more_bitmaps_than_its_array_holds():
    dev = torch.device("cuda:0")
    G = 65
    off = np.zeros(G + 1, dtype=np.int64)
    bits = torch.zeros(G * 32, dtype=torch.int32, device=dev)
    res = torch.zeros(64, dtype=torch.uint8, device=dev)
    capi.lib.rt_scan_slots_static.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint32,
                                              C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]
    status = capi.lib.rt_scan_slots_static(None, off.ctypes.data, G, 8191, 1024, 8, bits.data_ptr(),
                                           res.data_ptr(), None)
    assert status == capi.RT_ERR_CAPACITY
    assert "static scratch" in capi.strerror(status)
