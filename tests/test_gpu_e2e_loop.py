"""GPU: the end-to-end loop on real managed memory, small -- every decode step
plans from that step's slot table, hands the ranges to the prefetch executor
and runs the paged decode-attention reader over the same slots.

Checked at every step: the ranges equal the oracle's (the restated reference
chain on the same ids, from the same record of what is resident); after the
job, the driver reports every planned range at the destination the plan named;
the reader's output over the migrated pages equals a NumPy fp32 reference."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import compose
from retarget_b200 import capi, workloads
from retarget_b200.planner import DevicePlanner, ranges_from_tensor, ranges_to_tuples, result_from_tensor

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

MIB = 1 << 20


from retarget_b200.capi import UvmConfig  # noqa: E402


def test_plan_prefetch_attention_every_step():
    os.environ.pop("RETARGET_B200_LIBCUDA", None)
    from cuda.bindings import driver as cu
    from cuda.bindings import runtime as cudart
    dev = torch.device("cuda:0")
    torch.zeros(1, device=dev)
    err, ok = cudart.cudaDeviceGetAttribute(cudart.cudaDeviceAttr.cudaDevAttrConcurrentManagedAccess, 0)
    if int(err) or not ok:
        pytest.skip("no concurrent managed access on this device")
    lib = capi.lib
    layers, heads, bytes_per_slot, pool_slots = 2, 8, 2048, 8192
    layout = workloads.Layout(layers, bytes_per_slot, pool_slots)          # 16 MiB per buffer, 8 blocks, one bitmap
    alloc, budget = layout.alloc_bytes, 5
    trace = workloads.decode_trace(3, steps=14, pool_slots=pool_slots, arrival_rate=0.6, median=400,
                                   mean_output=6, initial_requests=5, shuffle_pages=False)
    err, ctx = cu.cuCtxGetCurrent()
    rng = np.random.default_rng(8)
    ptrs, host_views = [], []
    for _ in range(2 * layers):
        err, p = cudart.cudaMallocManaged(alloc, cudart.cudaMemAttachGlobal)
        assert int(err) == 0
        ptrs.append(int(p))
        view = np.ctypeslib.as_array((C.c_uint16 * (alloc // 2)).from_address(int(p)))
        # random bf16 values in (-2, 2): sign, exponent 0x3c..0x3f, random mantissa
        view[:] = (rng.integers(0, 2, alloc // 2, dtype=np.uint16) << 15) | \
                  (rng.integers(0x3c00, 0x4000, alloc // 2, dtype=np.uint16))
        host_views.append(view)
    lib.rt_uvm_register.argtypes = [C.c_uint64, C.c_uint64, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_uint64)]
    lib.rt_uvm_unregister_ptr.argtypes = [C.c_uint64]
    lib.rt_uvm_submit_ranges.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.POINTER(C.c_uint64)]
    lib.rt_uvm_wait.argtypes = [C.c_uint64, C.c_double, C.POINTER(C.c_int)]
    lib.rt_paged_attention.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p]
    cfg = UvmConfig(None, 2 * MIB, 8 * MIB, 2, 0)
    capi.check(lib.rt_uvm_start(C.byref(cfg)), "rt_uvm_start")
    planner = None
    try:
        ids = []
        for p in ptrs:
            i = C.c_uint64()
            capi.check(lib.rt_uvm_register(p, alloc, C.c_void_p(int(ctx)), 0, 1, C.byref(i)), "register")
            ids.append(i.value)
        id_arr = (C.c_uint64 * len(ids))(*ids)
        planner = DevicePlanner(layout, 0)
        resident = [set()]
        d_out = torch.zeros(1024 * 24, dtype=torch.uint8, device=dev)
        d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
        d_k = torch.tensor(ptrs[:layers], dtype=torch.int64, device=dev)
        d_v = torch.tensor(ptrs[layers:], dtype=torch.int64, device=dev)
        moved_any = evicted_any = False
        for step, t in enumerate(trace):
            n = len(t.read_slots)
            off = np.array([0, n], np.int64)
            batch = workloads.SlotBatch(layout, t.read_slots, off, t.req_off, budget)
            want, info = compose.plan_step(batch, resident, evict=True, literal=True)
            d_slots = torch.from_numpy(t.read_slots).to(dev)
            planner.step_device(d_slots, off, budget, capi.RT_PLAN_EVICT, d_out, d_res)
            planner.sync()
            res = result_from_tensor(d_res)
            ranges = ranges_from_tensor(d_out, res["n_ranges"])
            assert res["flags"] == 0 and ranges_to_tuples(ranges) == want, step
            if len(ranges):
                job, cuda_err = C.c_uint64(), C.c_int()
                keep = np.ascontiguousarray(ranges)
                capi.check(lib.rt_uvm_submit_ranges(keep.ctypes.data, len(keep), id_arr, len(ids), C.byref(job)),
                           "rt_uvm_submit_ranges")
                capi.check(lib.rt_uvm_wait(job.value, 60.0, C.byref(cuda_err)), "rt_uvm_wait")
                assert cuda_err.value == 0
                for buf, dst, offset, nbytes in want:
                    err, where = cudart.cudaMemRangeGetAttribute(
                        4, cudart.cudaMemRangeAttribute.cudaMemRangeAttributeLastPrefetchLocation,
                        ptrs[buf] + offset, nbytes)
                    assert int(err) == 0 and int(where) == dst, (step, buf, dst, offset)
                moved_any |= info["blocks_added"] > 0
                evicted_any |= info["blocks_evicted"] > 0
            # the reader over this step's slots; one (request, layer, head) checked against NumPy
            live = t.live
            if not live:
                continue
            q = (torch.randn(live, layers, heads, 128, device=dev) * 0.5).to(torch.bfloat16)
            out = torch.zeros(live, layers, heads, 128, dtype=torch.float32, device=dev)
            d_off = torch.from_numpy(t.req_off).to(dev)
            st = lib.rt_paged_attention(d_k.data_ptr(), d_v.data_ptr(), layers, heads, q.data_ptr(),
                                        d_slots.data_ptr(), d_off.data_ptr(), live, layout.capacity,
                                        out.data_ptr(), None)
            assert st == 0
            torch.cuda.synchronize()
            r, l, h = step % live, step % layers, step % heads
            ids_r = t.read_slots[t.req_off[r]:t.req_off[r + 1]]

            def rows(view):
                raw = np.stack([view[s * 1024 + h * 128: s * 1024 + (h + 1) * 128] for s in ids_r])
                return (raw.astype(np.uint32) << 16).view(np.float32)
            k, v = rows(host_views[l]), rows(host_views[layers + l])
            s = (k @ q[r, l, h].float().cpu().numpy()) / np.sqrt(128.0)
            p = np.exp(s - s.max())
            np.testing.assert_allclose(out[r, l, h].cpu().numpy(), (p / p.sum()) @ v, rtol=1e-2, atol=1e-3)
        assert moved_any and evicted_any
    finally:
        capi.check(lib.rt_uvm_stop(), "rt_uvm_stop")
        if planner is not None:
            planner.close()
        for p in ptrs:
            lib.rt_uvm_unregister_ptr(p)
            cudart.cudaFree(p)
