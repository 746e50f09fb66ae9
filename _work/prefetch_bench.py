"""Prefetch experiment on real managed memory (scaled-down form of the
oversubscribed end-to-end configuration).

    python -m retarget_b200.prefetch_bench [--buffers 8] [--gib-per-buffer 1]

What it measures, on one GPU, and prints as one JSON document:

* host link: pinned host -> device copy bandwidth (the yardstick);
* executor: GB/s of whole-registry migrations (everything to the CPU, everything
  to the GPU) through the UVM server, for a reference-like setting (one stream,
  one wait per 16 MiB or 256 MiB chunk -- the reference also creates and
  destroys a stream per chunk) and for the batched multi-stream default;
* plan -> prefetch -> read: a paged reader kernel touches the K/V rows of the
  live slots in every buffer, once with all pages on the CPU (demand faults)
  and once after the placement plan's ranges were prefetched.

The full configuration (160 GiB of KV + 20 GiB ballast, oversubscribing the
GPU) is deliberately not run: it would need ~180 GiB of host memory on a shared
machine.  Pages are pushed to the CPU explicitly between trials instead.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import time

import numpy as np

MIB = 1 << 20
GIB = 1 << 30


class UvmConfig(C.Structure):
    _fields_ = [("socket_path", C.c_char_p), ("chunk_bytes", C.c_uint64), ("batch_bytes", C.c_uint64),
                ("streams", C.c_uint32), ("listen", C.c_int32)]


class UmCounters:
    """GPU page-fault groups and migrated bytes from CUPTI's unified-memory
    activity records, when libretarget_umcount.so was built and CUPTI agrees."""
    NAMES = ("gpu_page_fault_groups", "cpu_page_faults", "bytes_host_to_device", "bytes_device_to_host",
             "records", "records_dropped")

    def __init__(self):
        from pathlib import Path
        self.ok, self.why, self.lib = False, "", None
        path = Path(__file__).resolve().parent / "libretarget_umcount.so"
        if not path.exists():
            self.why = "libretarget_umcount.so was not built (no CUPTI in the toolkit)"
            return
        try:
            self.lib = C.CDLL(str(path))
        except OSError as e:
            self.why = f"cannot load the CUPTI helper: {e}"
            return
        self.lib.rt_um_counters_error.restype = C.c_char_p
        if self.lib.rt_um_counters_enable() != 0:
            self.why = self.lib.rt_um_counters_error().decode()
            return
        self.ok = True
        self.kinds = int(self.lib.rt_um_counters_kinds())

    def read(self):
        if not self.ok:
            return None
        buf = (C.c_uint64 * 6)()
        if self.lib.rt_um_counters_read(buf) != 0:
            self.ok, self.why = False, self.lib.rt_um_counters_error().decode()
            return None
        got = dict(zip(self.NAMES, (int(v) for v in buf)))
        if self.kinds < 4:
            got["cpu_page_faults"] = None
        if self.kinds < 3:
            got["gpu_page_fault_groups"] = None
        return got

    def close(self):
        if self.ok:
            self.lib.rt_um_counters_disable()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--buffers", type=int, default=8)
    ap.add_argument("--gib-per-buffer", type=float, default=1.0)
    ap.add_argument("--requests", type=int, default=128)
    args = ap.parse_args()

    import torch
    from cuda.bindings import driver as cu
    from cuda.bindings import runtime as cudart
    from retarget_b200 import capi, workloads
    from retarget_b200.control import LocalUvm
    from retarget_b200.planner import DevicePlanner, ranges_from_tensor, result_from_tensor

    lib = capi.lib
    dev = torch.device("cuda:0")
    # the counters are switched on between driver initialisation and the first context
    cu.cuInit(0)
    counters = UmCounters()
    torch.cuda.set_device(0)
    torch.zeros(1, device=dev)
    out = {"gpu": torch.cuda.get_device_name(0)}
    err, concurrent = cudart.cudaDeviceGetAttribute(cudart.cudaDeviceAttr.cudaDevAttrConcurrentManagedAccess, 0)
    if int(err) != 0 or not concurrent:
        print(json.dumps({"unavailable": "device has no concurrent managed access"}))
        return

    # ---- yardstick: pinned host -> device copies ----
    n = 1 << 30
    host = torch.empty(n, dtype=torch.uint8).pin_memory()
    devbuf = torch.empty(n, dtype=torch.uint8, device=dev)
    for _ in range(2):
        devbuf.copy_(host, non_blocking=True)
    torch.cuda.synchronize()
    t = time.perf_counter()
    for _ in range(4):
        devbuf.copy_(host, non_blocking=True)
    torch.cuda.synchronize()
    h2d = 4 * n / (time.perf_counter() - t) / 1e9
    t = time.perf_counter()
    for _ in range(4):
        host.copy_(devbuf, non_blocking=True)
    torch.cuda.synchronize()
    d2h = 4 * n / (time.perf_counter() - t) / 1e9
    out["host_link_gbs"] = {"h2d_pinned": h2d, "d2h_pinned": d2h}
    del host, devbuf

    # ---- managed KV buffers, registered with the in-process UVM server ----
    bytes_per_slot = 2048
    alloc = int(args.gib_per_buffer * GIB) // (2 * MIB) * (2 * MIB)
    layers = args.buffers // 2
    pool_slots = alloc // bytes_per_slot
    err, ctx = cu.cuCtxGetCurrent()
    assert int(err) == 0
    ptrs = []
    for _ in range(args.buffers):
        err, p = cudart.cudaMallocManaged(alloc, cudart.cudaMemAttachGlobal)
        assert int(err) == 0, err
        ptrs.append(int(p))
        cudart.cudaMemset(p, 0x11, alloc)          # first touch on the GPU
    torch.cuda.synchronize()
    lib.rt_uvm_register.argtypes = [C.c_uint64, C.c_uint64, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_uint64)]
    ids = []
    for p in ptrs:
        i = C.c_uint64()
        capi.check(lib.rt_uvm_register(p, alloc, C.c_void_p(int(ctx)), 0, 1, C.byref(i)), "register")
        ids.append(i.value)
    total = alloc * args.buffers
    uvm = LocalUvm()

    def run_job(line):
        t0 = time.perf_counter()
        reply = uvm.command(line)
        assert reply.get("ok"), reply
        uvm._wait_job(reply["job_id"], timeout=600, poll_seconds=0.0005)
        return time.perf_counter() - t0

    settings = [("reference-like: 1 stream, wait per 16 MiB chunk", 16 * MIB, 16 * MIB, 1),
                ("reference-like: 1 stream, wait per 256 MiB chunk", 256 * MIB, 256 * MIB, 1),
                ("batched: 4 streams, 16 MiB chunks, wait per 256 MiB", 16 * MIB, 256 * MIB, 4),
                ("batched: 4 streams, 64 MiB chunks, wait per 1 GiB", 64 * MIB, 1024 * MIB, 4)]
    out["executor"] = []
    for name, chunk, batch, streams in settings:
        cfg = UvmConfig(None, chunk, batch, streams, 0)
        capi.check(lib.rt_uvm_start(C.byref(cfg)), "rt_uvm_start")
        gen = uvm.status().allocation_generation
        run_job(f"targetv {gen} {total}")               # everything on the GPU first
        to_cpu = run_job(f"targetv {gen} 0")
        to_gpu = run_job(f"targetv {gen} {total}")
        out["executor"].append({"setting": name, "to_cpu_gbs": total / to_cpu / 1e9,
                                "to_gpu_gbs": total / to_gpu / 1e9,
                                "to_gpu_frac_of_h2d_link": total / to_gpu / 1e9 / h2d})
        capi.check(lib.rt_uvm_stop(), "rt_uvm_stop")

    # ---- plan -> prefetch -> read ----
    cfg = UvmConfig(None, 64 * MIB, 1024 * MIB, 4, 0)
    capi.check(lib.rt_uvm_start(C.byref(cfg)), "rt_uvm_start")
    gen = uvm.status().allocation_generation
    layout = workloads.Layout(layers, bytes_per_slot, pool_slots)
    rng = np.random.default_rng(0)
    pool = workloads.PagePool(pool_slots, rng)
    lens = workloads.request_lengths(rng, args.requests, 8192, hi=32768)
    # keep the live set to about a quarter of the pool, as a 25 % budget would
    lens = (lens * min(1.0, 0.25 * pool_slots / lens.sum())).astype(np.int64)
    slots = np.concatenate(workloads.admit(pool, lens)).astype(np.int64)
    d_slots = torch.from_numpy(slots).to(dev)
    d_ptrs = torch.tensor(ptrs, dtype=torch.int64, device=dev)
    d_sums = torch.zeros(args.buffers, dtype=torch.int64, device=dev)
    lib.rt_paged_read.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint64,
                                  C.c_void_p, C.c_void_p]
    stream = torch.cuda.Stream(device=dev)

    def read_once():
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        capi.check(lib.rt_paged_read(d_ptrs.data_ptr(), args.buffers, bytes_per_slot, d_slots.data_ptr(),
                                     len(slots), layout.capacity, d_sums.data_ptr(), stream.cuda_stream), "read")
        stream.synchronize()
        return time.perf_counter() - t0, d_sums.cpu().numpy().copy()

    read_bytes = len(slots) * bytes_per_slot * args.buffers
    run_job(f"targetv {gen} 0")
    counters.read()                                    # drop what the set-up caused
    t_fault, sums_fault = read_once()                  # every page faults in
    um_fault = counters.read()
    t_warm, _ = read_once()                            # now resident
    run_job(f"targetv {gen} 0")
    planner = DevicePlanner(layout, 0)
    d_out = torch.zeros((1 << 14) * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    t0 = time.perf_counter()
    planner.step_device(d_slots, np.array([0, len(slots)], np.int64), layout.n_blocks, 0, d_out, d_res,
                        stream.cuda_stream)
    stream.synchronize()
    res = result_from_tensor(d_res)
    ranges = ranges_from_tensor(d_out, res["n_ranges"]).copy()
    t_plan = time.perf_counter() - t0
    lib.rt_uvm_submit_ranges.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.POINTER(C.c_uint64)]
    lib.rt_uvm_wait.argtypes = [C.c_uint64, C.c_double, C.POINTER(C.c_int)]
    id_arr = (C.c_uint64 * len(ids))(*ids)
    job, cuda_err = C.c_uint64(), C.c_int()
    t0 = time.perf_counter()
    capi.check(lib.rt_uvm_submit_ranges(ranges.ctypes.data, len(ranges), id_arr, len(ids), C.byref(job)), "submit")
    capi.check(lib.rt_uvm_wait(job.value, 600.0, C.byref(cuda_err)), "wait")
    t_prefetch = time.perf_counter() - t0
    um_prefetch = counters.read()
    t_after, sums_after = read_once()
    um_after = counters.read()
    out["plan_prefetch_read"] = {
        "buffers": args.buffers, "alloc_bytes": alloc, "live_slots": int(len(slots)),
        "rows_read_bytes": read_bytes, "plan_ranges": int(res["n_ranges"]),
        "plan_bytes": int(res["gpu_bytes"]), "plan_seconds": t_plan,
        "prefetch_seconds": t_prefetch, "prefetch_gbs": res["gpu_bytes"] / t_prefetch / 1e9,
        "prefetch_frac_of_h2d_link": res["gpu_bytes"] / t_prefetch / 1e9 / h2d,
        "read_seconds_pages_on_cpu": t_fault, "read_seconds_after_plan": t_after,
        "read_seconds_resident": t_warm, "checksums_equal": bool(np.array_equal(sums_fault, sums_after)),
        "um_counters": {"reader_pages_on_cpu": um_fault, "prefetch_of_the_plan": um_prefetch,
                        "reader_after_plan": um_after} if counters.ok else f"unavailable ({counters.why})"}
    counters.close()
    capi.check(lib.rt_uvm_stop(), "rt_uvm_stop")
    planner.close()
    # ---- incremental window moves: every step evicts one stride and grows one stride per buffer ----
    # (the reference's incremental update, select.cpp:24231-24240; CPU-bound ranges are waited for
    # before the GPU-bound ones.  Letting the two directions overlap was tried and gained nothing:
    # the driver runs the migrations of one process one after the other.)
    cfg = UvmConfig(None, 16 * MIB, 256 * MIB, 4, 0)
    capi.check(lib.rt_uvm_start(C.byref(cfg)), "rt_uvm_start")
    gen = uvm.status().allocation_generation
    width, stride, big = alloc // 4, alloc // 8, (1 << 64) - 1
    run_job(f"windowv {gen} {alloc} {args.buffers} {big} {big} 0 {width}")
    lo, times = 0, []
    for _ in range(5):
        times.append(run_job(f"windowv {gen} {alloc} {args.buffers} {lo} {lo + width} "
                             f"{lo + stride} {lo + stride + width}"))
        lo += stride
    out["window_moves"] = {"bytes_each_way_per_step": stride * args.buffers, "seconds_per_step_best": min(times),
                           "seconds_per_step_median": sorted(times)[2],
                           "gbs_both_directions": 2 * stride * args.buffers / min(times) / 1e9}
    capi.check(lib.rt_uvm_stop(), "rt_uvm_stop")
    for p in ptrs:
        cudart.cudaFree(p)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
