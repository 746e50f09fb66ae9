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


from retarget_b200.capi import UvmConfig  # noqa: E402


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
        before = uvm.status()                  # the byte counters run for the life of the process
        reply = uvm.command(f"windowv {gen} {size} 4 {big} {big} {2 * MIB} {6 * MIB}")
        assert reply["ok"], reply
        st = uvm._wait_job(reply["job_id"], timeout=60, poll_seconds=0.002)
        assert st.last_error == 0
        assert st.completed_gpu_bytes - before.completed_gpu_bytes == 4 * 4 * MIB
        assert st.completed_cpu_bytes - before.completed_cpu_bytes == 4 * 4 * MIB
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


def test_probe_to_prefetch_chain(managed, tmp_path, monkeypatch):
    """The whole event-driven path on real managed memory: probe events on the
    device -> published snapshot -> the scheduler-side controller -> blocksv on
    the control protocol -> the executor's cuMemPrefetchAsync calls.  The blocks
    the policy picks end up with the GPU as their last prefetch location in
    every buffer; nothing else was touched."""
    import time
    cudart, ctx, ptrs, size = managed
    from retarget_b200 import capi
    from retarget_b200.cache_window import CacheWindowSpec
    from retarget_b200.control import LocalUvm
    from retarget_b200.probe import DeviceWriter
    from retarget_b200.slot_placement import SlotPlacementController, SlotPlacementSpec
    lib = capi.lib
    lib.rt_uvm_register.argtypes = [C.c_uint64, C.c_uint64, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_uint64)]
    lib.rt_uvm_unregister_ptr.argtypes = [C.c_uint64]
    slot_bytes, block_tokens = 2048, 256
    capacity = size // slot_bytes - 1                       # 4095 slots, 16 blocks of 512 KiB
    block_bytes = slot_bytes * block_tokens
    monkeypatch.setenv("RETARGET_SLOT_FEEDBACK_DIR", str(tmp_path))
    dev = torch.device("cuda:0")
    cfg = UvmConfig(None, 2 * MIB, 6 * MIB, 2, 0)
    capi.check(lib.rt_uvm_start(C.byref(cfg)), "start")
    writer = None
    try:
        for p in ptrs:
            capi.check(lib.rt_uvm_register(p, size, C.c_void_p(ctx), 0, 1, None), "register")
        uvm = LocalUvm()
        gen, _ = uvm._allocation_snapshot()
        # everything to the CPU first, so that a GPU location afterwards is the plan's doing
        reply = uvm.command(f"targetv {gen} 0")
        uvm._wait_job(reply["job_id"], timeout=60, poll_seconds=0.002)
        writer = DeviceWriter(pid=os.getpid(), block_tokens=block_tokens, buffers=len(ptrs), slot_bytes=slot_bytes)
        held = torch.arange(1, 700, dtype=torch.int64, device=dev)                 # blocks 0..2
        writer.submit("alloc", {"slot": held, "free_head": torch.arange(3000, 3100, dtype=torch.int64, device=dev)},
                      allocator_size=capacity, need_sort=False)
        reads = torch.cat([torch.arange(1, 300, device=dev), torch.arange(2600, 2700, device=dev)]).to(torch.int32)
        writer.submit("attention", {"read": reads, "write": torch.tensor([699], dtype=torch.int64, device=dev)},
                      path="eager", mode="DECODE", batch_size=2, reads="all_cached_kv")
        writer.publish(writer.feedback.at)
        spec = CacheWindowSpec(size, len(ptrs), slot_bytes, 4 * block_tokens, block_tokens, block_tokens)
        ctl = SlotPlacementController(spec, SlotPlacementSpec(block_tokens=block_tokens, max_blocks_per_update=4),
                                      os.getpid())
        assert ctl.budget == 4
        now = time.monotonic()
        snap = ctl.snapshot(now)
        desired, selected = ctl.choose(snap, now)
        # reads: blocks 0, 1 and 10; writes: block 2 (the write stamp of the attention event); then the free head
        assert desired == [0, 1, 10, 2] and selected == desired
        result = ctl.update(uvm, {}, now)
        assert result is not None and uvm.status().last_error == 0
        assert uvm.status().job_completed_bytes == len(ptrs) * 4 * block_bytes
        for p in ptrs:
            for b in range(16):
                where = last_location(cudart, p + b * block_bytes, block_bytes)
                assert where == (0 if b in desired else -1), (b, where)
        # a second update with nothing new to move sends nothing
        assert ctl.update(uvm, {}, time.monotonic()) is None
    finally:
        if writer is not None:
            writer.close()
        for p in ptrs:
            lib.rt_uvm_unregister_ptr(p)
        lib.rt_uvm_stop()


def test_window_controller_moves_the_window(managed):
    """The counter-driven path on real managed memory: Prometheus counters ->
    CacheWindowController.update -> windowv on the control protocol -> executor.
    After every accepted update the window's bytes were last sent to the GPU and
    everything outside it to the CPU, in every buffer."""
    cudart, ctx, ptrs, size = managed
    from retarget_b200 import capi
    from retarget_b200.cache_window import CacheWindowController, CacheWindowSpec
    from retarget_b200.control import LocalUvm
    lib = capi.lib
    lib.rt_uvm_register.argtypes = [C.c_uint64, C.c_uint64, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_uint64)]
    lib.rt_uvm_unregister_ptr.argtypes = [C.c_uint64]
    spec = CacheWindowSpec(size, len(ptrs), 2048, 1024, 512, 512, min_update_seconds=1.0, idle_only=True)
    ctl = CacheWindowController(spec)
    cfg = UvmConfig(None, 1 * MIB, 4 * MIB, 2, 0)
    capi.check(lib.rt_uvm_start(C.byref(cfg)), "start")

    def metrics(prompt, generated, running=0, queued=0):
        return {"sglang:prompt_tokens_total": float(prompt), "sglang:generation_tokens_total": float(generated),
                "sglang:num_running_reqs": float(running), "sglang:num_queue_reqs": float(queued)}

    def check(window):
        lo, hi = window
        for p in ptrs:
            if lo:
                assert last_location(cudart, p, lo) == -1
            assert last_location(cudart, p + lo, hi - lo) == 0
            if hi < size:
                assert last_location(cudart, p + hi, size - hi) == -1

    try:
        for p in ptrs:
            capi.check(lib.rt_uvm_register(p, size, C.c_void_p(ctx), 0, 1, None), "register")
        uvm = LocalUvm()
        first = ctl.update(uvm, metrics(100, 0), 10.0, initial=True)
        assert first["initial"] and first["new_window"] == [0, 2 * MIB]
        assert first["requested_gpu_bytes"] == len(ptrs) * 2 * MIB
        assert first["requested_cpu_bytes"] == len(ptrs) * (size - 2 * MIB)
        check(first["new_window"])
        assert ctl.update(uvm, metrics(700, 200, running=2), 12.0) is None          # not idle
        moved = ctl.update(uvm, metrics(700, 200), 12.5)
        assert moved["old_window"] == [0, 2 * MIB] and moved["new_window"] == [1 * MIB, 3 * MIB]
        assert moved["requested_gpu_bytes"] == moved["requested_cpu_bytes"] == len(ptrs) * MIB
        check(moved["new_window"])
        assert ctl.update(uvm, metrics(3000, 500), 12.9) is None                    # too soon
        far = ctl.update(uvm, metrics(3000, 500), 14.0)
        assert far["new_window"] == [6 * MIB, 8 * MIB]
        check(far["new_window"])
        assert uvm.status().last_error == 0
    finally:
        for p in ptrs:
            lib.rt_uvm_unregister_ptr(p)
        lib.rt_uvm_stop()
