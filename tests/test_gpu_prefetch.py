"""Real-driver checks on a GPU: the UVM server's executor against managed
memory (the prefetch calls really land where the plan says) and the paged
reader kernel against a numpy checksum."""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

MIB = 1 << 20


class UvmConfig(C.Structure):
    _fields_ = [("socket_path", C.c_char_p), ("chunk_bytes", C.c_uint64), ("batch_bytes", C.c_uint64),
                ("streams", C.c_uint32), ("listen", C.c_int32)]


@pytest.fixture()
def managed():
    os.environ.pop("RETARGET_B200_LIBCUDA", None)
    from cuda.bindings import driver as cu
    from cuda.bindings import runtime as cudart
    torch.zeros(1, device="cuda:0")
    err, ok = cudart.cudaDeviceGetAttribute(cudart.cudaDeviceAttr.cudaDevAttrConcurrentManagedAccess, 0)
    if int(err) or not ok:
        pytest.skip("no concurrent managed access on this device")
    err, ctx = cu.cuCtxGetCurrent()
    n, size = 4, 8 * MIB
    ptrs = []
    for _ in range(n):
        err, p = cudart.cudaMallocManaged(size, cudart.cudaMemAttachGlobal)
        assert int(err) == 0
        ptrs.append(int(p))
    yield cudart, int(ctx), ptrs, size
    for p in ptrs:
        cudart.cudaFree(p)


def last_location(cudart, ptr, nbytes):
    err, value = cudart.cudaMemRangeGetAttribute(
        4, cudart.cudaMemRangeAttribute.cudaMemRangeAttributeLastPrefetchLocation, ptr, nbytes)
    assert int(err) == 0, err
    return int(value)


def test_paged_reader_checksum(managed):
    cudart, ctx, ptrs, size = managed
    from retarget_b200 import capi
    rng = np.random.default_rng(4)
    views = []
    for p in ptrs:
        host = np.ctypeslib.as_array((C.c_uint16 * (size // 2)).from_address(p))
        host[:] = rng.integers(0, 1 << 16, size // 2, dtype=np.uint16)
        views.append(host)
    bytes_per_slot, capacity = 2048, size // 2048 - 1
    slots = rng.integers(-3, capacity + 4, 3000).astype(np.int64)
    valid = slots[(slots >= 1) & (slots <= capacity)]
    want = [int(sum(int(v[s * 1024:(s + 1) * 1024].astype(np.uint64).sum()) for s in valid)) for v in views]
    dev = torch.device("cuda:0")
    d_slots = torch.from_numpy(slots).to(dev)
    d_ptrs = torch.tensor(ptrs, dtype=torch.int64, device=dev)
    d_sums = torch.zeros(len(ptrs), dtype=torch.int64, device=dev)
    capi.lib.rt_paged_read.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint64,
                                       C.c_void_p, C.c_void_p]
    stream = torch.cuda.Stream(device=dev)
    capi.check(capi.lib.rt_paged_read(d_ptrs.data_ptr(), len(ptrs), bytes_per_slot, d_slots.data_ptr(),
                                      len(slots), capacity, d_sums.data_ptr(), stream.cuda_stream), "read")
    stream.synchronize()
    assert d_sums.cpu().numpy().astype(np.uint64).tolist() == want


def test_executor_moves_managed_ranges(managed):
    cudart, ctx, ptrs, size = managed
    from retarget_b200 import capi
    from retarget_b200.control import LocalUvm
    lib = capi.lib
    lib.rt_uvm_register.argtypes = [C.c_uint64, C.c_uint64, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_uint64)]
    lib.rt_uvm_unregister_ptr.argtypes = [C.c_uint64]
    cfg = UvmConfig(None, 2 * MIB, 6 * MIB, 2, 0)
    capi.check(lib.rt_uvm_start(C.byref(cfg)), "start")
    try:
        for p in ptrs:
            capi.check(lib.rt_uvm_register(p, size, C.c_void_p(ctx), 0, 1, None), "register")
        uvm = LocalUvm()
        gen, allocs = uvm._allocation_snapshot()
        assert [a["bytes"] for a in allocs] == [size] * 4
        big = (1 << 64) - 1
        reply = uvm.command(f"windowv {gen} {size} 4 {big} {big} {2 * MIB} {6 * MIB}")
        assert reply["ok"], reply
        st = uvm._wait_job(reply["job_id"], timeout=60, poll_seconds=0.002)
        assert st.last_error == 0
        assert st.completed_gpu_bytes == 4 * 4 * MIB and st.completed_cpu_bytes == 4 * 4 * MIB
        for p in ptrs:
            assert last_location(cudart, p, 2 * MIB) == -1                     # cudaCpuDeviceId
            assert last_location(cudart, p + 2 * MIB, 4 * MIB) == 0
            assert last_location(cudart, p + 6 * MIB, 2 * MIB) == -1
        reply = uvm.command(f"windowv {gen} {size} 4 {2 * MIB} {6 * MIB} {4 * MIB} {8 * MIB}")
        st = uvm._wait_job(reply["job_id"], timeout=60, poll_seconds=0.002)
        assert st.last_error == 0 and st.job_completed_bytes == 4 * 4 * MIB
        for p in ptrs:
            assert last_location(cudart, p + 2 * MIB, 2 * MIB) == -1
            assert last_location(cudart, p + 6 * MIB, 2 * MIB) == 0
        # the data survived the round trips
        host = np.ctypeslib.as_array((C.c_uint8 * 64).from_address(ptrs[0] + 5 * MIB))
        host[:] = 7
        reply = uvm.command(f"prefetch {allocs[0]['id']} {4 * MIB} {2 * MIB} gpu")
        uvm._wait_job(reply["job_id"], timeout=60, poll_seconds=0.002)
        reply = uvm.command(f"prefetch {allocs[0]['id']} {4 * MIB} {2 * MIB} cpu")
        uvm._wait_job(reply["job_id"], timeout=60, poll_seconds=0.002)
        assert host.tolist() == [7] * 64
    finally:
        for p in ptrs:
            lib.rt_uvm_unregister_ptr(p)
        lib.rt_uvm_stop()
