#!/usr/bin/env python3
"""Placement-plan benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
                    [--launch graph|stream] [--unchained] [--tma] [--no-cpu] [--no-extras]

One step = one placement plan for one decode step of the headline workload:
40 layers (80 KV buffers of 512 MiB), 256 requests, a 262,144-slot pool, and per
(layer, request) touched sets of the newest 128 slots plus 2048 Zipf(1.1)
history draws -- 22.3 M int64 slot ids (178 MB) per step.  Two different
batches alternate, so every step re-reads more than the L2 holds; one lives in
the lower half of every buffer and one in the upper half, so every plan evicts
one run and adds one run per buffer (160 ranges per step, the shape of the
reference's incremental window update).

The JSON line (rank 0) carries every term of the metric:

`value`      device time per step, slot ids already in HBM: two CUDA events on
             the launching stream around the timed steps, max over ranks.  The
             steps go out as replays of a CUDA graph of 100 chained steps; the graph
             is replayed until the timed region lasts at least 50 ms, so that
             `--steps 20` does not end up timing 0.6 ms (`timed_steps` says how
             many steps were timed; `steps` stays the number asked for)
`roofline`   slot-scan GB/s of that step against the measured HBM copy peak
`e2e`        the same plan through the host-buffer C-ABI call: pinned host ids
             are copied to the device, planned, the range list comes back
`prefetch`   GB/s of the prefetch executor on managed memory against the pinned
             host link, measured in the same run (one GPU)
`feedback`   the event-driven path (device-resident feedback state) on an
             incremental decode trace, beside the Python chain on one core
`configs`    the other stated configurations (full refresh, sparse feedback,
             one tensor-parallel shard): us, GB/s, fraction of the peak
`tp_shard_us`  (every N) the tensor-parallel shard configuration per rank

--workload e2e_prefetch  the end-to-end loop on managed memory: every decode step
             plans from that step's slot table, hands the ranges to the prefetch
             executor and runs a paged decode-attention reader; with the plan,
             with evictions only, and with everything resident

--impl reference  times the CPU restatement of the reference's Python path on
             the host cores: every step runs all layers, one process per core
"""
from __future__ import annotations

import argparse
import ctypes as C
import dataclasses
import json
import math
import multiprocessing as mp
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "placement_plan_us_per_decode_step"
UNIT = "us/step"
FALLBACK_HBM_GBS = 6650.0
MIN_TIMED_MS = 50.0
MIB, GIB = 1 << 20, 1 << 30


def make_batches(name: str):
    """The two batches that alternate in the timed region."""
    from retarget_b200 import workloads
    if name == "target":
        return list(workloads.target_pair("moving"))
    if name in ("steady", "fragmented"):
        return list(workloads.target_pair(name))
    return [make_workload(name, 0), make_workload(name, 1)]


def make_workload(name: str, seed: int):
    from retarget_b200 import workloads
    if name == "sparse":
        return workloads.sparse_feedback(seed)
    if name == "full_refresh":
        return workloads.full_refresh(seed)
    if name == "tp_shard":
        return workloads.tp_shard(seed)
    raise SystemExit(f"unknown workload {name}")


def algorithmic_bytes(batch, n_ranges: int, id_bytes: int = 8) -> int:
    """Bytes one step must move: every slot id once, the group offsets, the
    resident words read and written, the ranges and the result record."""
    G = batch.layout.n_groups
    return id_bytes * batch.n_idx + 8 * (G + 1) + 2 * 4 * 32 * G + 24 * n_ranges + 64


def workload_config(batch, args) -> dict:
    """Describes the workload and how its steps are issued.  Both arms print the
    same dictionary for the same command line."""
    lay = batch.layout
    name = batch.name
    for tag, text in ((", lower half", ", steps alternate between the lower and upper half of every buffer"),
                      (", even blocks", ", steps alternate between even and odd blocks")):
        if name.endswith(tag):
            name = name[:-len(tag)] + text
    world = args.gpus
    if args.launch != "graph":
        launch = "one launch per step on the stream, >= 50 ms of steps"
    elif args.min_timed_ms >= 10:
        launch = f"CUDA graph of 100 steps, replayed until the timed region lasts >= {args.min_timed_ms:g} ms"
    else:
        launch = "CUDA graph of at most 20 steps, replayed once"
    if not args.unchained:
        launch += "; steps chained (programmatic dependent launch): the scan of step i+1 runs over the tail of step i"
    return {"workload": name, "layers": lay.layers, "kv_buffers": lay.n_buffers,
            "alloc_bytes": lay.alloc_bytes, "pool_slots": lay.pool_slots,
            "bytes_per_slot": lay.bytes_per_slot, "uvm_block_bytes": lay.block_bytes,
            "bitmaps": lay.n_groups, "blocks_per_bitmap": lay.n_blocks,
            "budget_blocks": batch.budget_blocks, "slot_ids_per_step": batch.n_idx,
            "slot_id_bytes_per_step": 8 * batch.n_idx, "index_dtype": "int64",
            "parallelism": f"{world} independent per-GPU planners (one KV shard each), no collective on the data path",
            "l2": f"{8 * batch.n_idx / 1e6:.0f} MB of ids per step, two batches alternate"
                  + (" (> 126 MB L2)" if 8 * batch.n_idx > 126e6 else " (fits the L2: a latency figure)"),
            "staging": "cp.async.bulk (TMA) -> shared" if args.tma else "ld.global 128-bit, two register sets",
            "gpu_arm_launch": launch,
            "reference_arm": "CPU restatement of the reference's Python chain, all layers of every step, "
                             "one process per host core",
            "evict": True}


# --------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons, power = [], [], set(), []
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0])); smax.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------
# CPU arms (oracle ports; the only place this file touches oracle/)
# --------------------------------------------------------------------------
_CPU = {}


def _cpu_layer(args):
    """Worker: the literal reference chain on one layer of one batch."""
    which, layer, resident_blocks = args
    from oracle import compose
    b = _CPU["batches"][which]
    lay = dataclasses.replace(b.layout, layers=1, shared_bitmap=True)
    lo, hi = int(b.group_off[layer]), int(b.group_off[layer + 1])
    ro = b.req_off
    k0, k1 = np.searchsorted(ro, lo, "left"), np.searchsorted(ro, hi, "right")
    from retarget_b200.workloads import SlotBatch
    one = SlotBatch(lay, b.slots[lo:hi], np.array([0, hi - lo], np.int64), ro[k0:k1] - lo,
                    b.budget_blocks)
    resident = [set(resident_blocks)]
    t = time.perf_counter()
    out, _ = compose.plan_step(one, resident, evict=True, literal=True)
    return time.perf_counter() - t, len(out), layer, sorted(resident[0])


def cpu_python_port(batches, layers, procs: int, steps: int, warmup: int):
    """The Python restatement of the reference path on the given layers of every
    step, spread over `procs` processes.  Returns the wall seconds of each timed
    step (for those layers; nothing is scaled here)."""
    _CPU["batches"] = batches
    resident = {}
    ctx = mp.get_context("fork")
    times = []
    with ctx.Pool(procs) as pool:
        for step in range(warmup + steps):
            t = time.perf_counter()
            res = pool.map(_cpu_layer, [(step % 2, l, resident.get(l, ())) for l in layers], chunksize=1)
            dt = time.perf_counter() - t
            for _, _, layer, blocks in res:
                resident[layer] = blocks
            if step >= warmup:
                times.append(dt)
    return times


def cpu_c_port(batches, reps: int):
    from oracle import c_oracle
    co = c_oracle.COracle(batches[0].layout)
    threads = min(co.max_threads, os.cpu_count() or 1)
    times = []
    for i in range(reps + 2):
        b = batches[i % 2]
        t = time.perf_counter()
        co.step(b.slots, b.group_off, b.budget_blocks, True, threads)
        if i >= 2:
            times.append(time.perf_counter() - t)
    return statistics.median(times), threads


def run_reference(args):
    """The reference arm: CPU only, rank 0 only.  Every step plans ALL layers."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    batches = make_batches(args.workload)
    cores = os.cpu_count() or 1
    L = batches[0].layout.n_groups
    procs = max(1, min(cores, L))
    t0 = time.perf_counter()
    times = cpu_python_port(batches, list(range(L)), procs, args.steps, args.warmup)
    wall = time.perf_counter() - t0
    per_step = statistics.mean(times)
    us = per_step * 1e6
    sample_text = (f"all {L} layers of every step through the Python restatement of "
                   f"encode_runs->blocks->target_blocks->choose->blocksv, {procs} processes; "
                   f"{args.steps} timed steps, nothing scaled")
    line = {"impl": "reference", "metric": METRIC, "value": us, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "int64",
            "data": "synthetic", "config": workload_config(batches[0], args),
            "cpu_baseline": {"value": us, "unit": UNIT, "cores": procs, "kind": "port", "sample": sample_text},
            "e2e": {"value": us, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "wall_s": wall}
    emit(line)


# --------------------------------------------------------------------------
# GPU arm: helpers
# --------------------------------------------------------------------------
class StepTimer:
    """Times back-to-back steps of one planner on one stream."""

    def __init__(self, torch, planner, stream, d_out, d_res, flags):
        self.torch, self.planner, self.stream = torch, planner, stream
        self.d_out, self.d_res, self.flags = d_out, d_res, flags

    def step(self, tensors, pair, i, handle=None, flags=None):
        b = pair[i % 2]
        self.planner.step_device(tensors[i % 2], b.group_off, b.budget_blocks,
                                 self.flags if flags is None else flags, self.d_out, self.d_res,
                                 handle if handle is not None else self.stream.cuda_stream)

    def result(self):
        from retarget_b200.planner import result_from_tensor
        r = result_from_tensor(self.d_res)
        if r["flags"]:
            raise SystemExit(f"bench.py: planner reported flags {r['flags']}")
        return r

    def timed(self, tensors, pair, *, min_steps, launch="graph", warm=4, min_ms=MIN_TIMED_MS, flags=None):
        """(us per step, steps timed, ranges of the last step).  Graph mode captures
        an even number of steps once and replays it."""
        torch = self.torch
        for i in range(warm):
            self.step(tensors, pair, i, flags=flags)
        torch.cuda.synchronize()
        self.result()
        per = 0
        graph = None
        if launch == "graph":
            # a replay's first step cannot chain to the replay before it: long graphs make that rare.
            # (runs that ask for no minimum time -- profiler captures -- keep the graph as short as the request)
            per = 100 if min_ms >= 10 else max(2, min(20, min_steps - min_steps % 2))
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream, capture_error_mode="thread_local"):
                for i in range(per):
                    self.step(tensors, pair, warm + i, torch.cuda.current_stream().cuda_stream, flags=flags)
            graph.replay()                    # untimed: first replay of a new graph
            torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]

        def run(n):
            ev[0].record(self.stream)
            if graph is not None:
                for _ in range(n // per):
                    graph.replay()
            else:
                for i in range(n):
                    self.step(tensors, pair, warm + i, flags=flags)
            ev[1].record(self.stream)
            torch.cuda.synchronize()
            return ev[0].elapsed_time(ev[1])

        unit = per if graph is not None else 2
        n = max(unit, -(-min_steps // unit) * unit)
        probe = run(n)                         # sizes the timed region, then it is measured afresh
        want = max(n, int(math.ceil(min_ms / max(probe / n, 1e-6))))
        n = -(-want // unit) * unit
        return n, run, graph


def upload(torch, dev, batches, dtype=None):
    return [torch.from_numpy(b.slots if dtype is None else b.slots.astype(dtype)).to(dev) for b in batches]


def prefetch_leg(torch, dev, gib: int = 4):
    """Prefetched GB/s against the host link: `gib` x 1 GiB managed buffers,
    registered with the in-process UVM server, moved as a whole to the CPU and
    back by the executor (64 MiB chunks on 4 side streams, one wait per GiB);
    the yardstick is a pinned host -> device copy measured just before."""
    from cuda.bindings import driver as cu
    from cuda.bindings import runtime as cudart
    from retarget_b200 import capi
    from retarget_b200.control import LocalUvm
    lib = capi.lib
    err, concurrent = cudart.cudaDeviceGetAttribute(cudart.cudaDeviceAttr.cudaDevAttrConcurrentManagedAccess,
                                                    dev.index or 0)
    if int(err) != 0 or not concurrent:
        return {"unavailable": "device has no concurrent managed access"}
    n = 1 << 30
    host = torch.empty(n, dtype=torch.uint8).pin_memory()
    devbuf = torch.empty(n, dtype=torch.uint8, device=dev)
    devbuf.copy_(host, non_blocking=True)
    torch.cuda.synchronize()
    t = time.perf_counter()
    for _ in range(3):
        devbuf.copy_(host, non_blocking=True)
    torch.cuda.synchronize()
    h2d = 3 * n / (time.perf_counter() - t) / 1e9
    del host, devbuf
    err, ctx = cu.cuCtxGetCurrent()
    ptrs = []
    for _ in range(gib):
        err, p = cudart.cudaMallocManaged(GIB, cudart.cudaMemAttachGlobal)
        if int(err) != 0:
            for q in ptrs:
                cudart.cudaFree(q)
            return {"unavailable": f"cudaMallocManaged failed: {err}"}
        ptrs.append(int(p))
        cudart.cudaMemset(p, 0x11, GIB)
    torch.cuda.synchronize()
    lib.rt_uvm_register.argtypes = [C.c_uint64, C.c_uint64, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_uint64)]
    lib.rt_uvm_unregister_ptr.argtypes = [C.c_uint64]
    for p in ptrs:
        capi.check(lib.rt_uvm_register(p, GIB, C.c_void_p(int(ctx)), dev.index or 0, 1, None), "rt_uvm_register")
    total = gib * GIB
    uvm = LocalUvm()
    cfg = capi.UvmConfig(None, 64 * MIB, 1024 * MIB, 4, 0)
    capi.check(lib.rt_uvm_start(C.byref(cfg)), "rt_uvm_start")
    try:
        gen = uvm.status().allocation_generation

        def job(line):
            t0 = time.perf_counter()
            reply = uvm.command(line)
            assert reply.get("ok"), reply
            done = uvm._wait_job(reply["job_id"], timeout=600, poll_seconds=0.0005)
            return time.perf_counter() - t0, done

        job(f"targetv {gen} {total}")
        to_cpu, _ = job(f"targetv {gen} 0")
        to_gpu, done = job(f"targetv {gen} {total}")
        out = {"h2d_link_gbs": h2d, "to_gpu_gbs": total / to_gpu / 1e9, "frac_of_link": total / to_gpu / 1e9 / h2d,
               "to_cpu_gbs": total / to_cpu / 1e9, "bytes_moved_each_way": total,
               "job_completed_bytes": done.job_completed_bytes,
               "executor": "64 MiB chunks on 4 side streams, one wait per GiB",
               "link_yardstick": "pinned host -> device copy of 1 GiB, same process, measured just before"}
        # a window that moves by its own width: half of every buffer goes to the CPU while the other half
        # comes in, first in the reference's order (all evictions, then all additions), then both at once
        half = GIB // 2
        job(f"windowfullv {gen} {GIB} {gib} 0 0 0 {half}")
        flips = [(0, half, half, GIB), (half, GIB, 0, half)]
        both = {}
        for name, overlap in (("in_order", 0), ("overlapped", 1)):
            capi.check(lib.rt_uvm_stop(), "rt_uvm_stop")
            cfg = capi.UvmConfig(None, 64 * MIB, 1024 * MIB, 4, 0, overlap)
            capi.check(lib.rt_uvm_start(C.byref(cfg)), "rt_uvm_start")
            spent = 0.0
            for k in range(6):
                o0, o1, n0, n1 = flips[k % 2]
                t, _ = job(f"windowv {gen} {GIB} {gib} {o0} {o1} {n0} {n1}")
                spent += t if k >= 4 else 0.0          # the first flips touch the host pages for the first time
            both[name + "_gbs"] = 2 * total / spent / 1e9
        both["bytes_per_plan"] = total
        both["what"] = ("windowv plans that evict one half of every buffer and bring in the other half: "
                        "GB/s over both directions together")
        out["both_ways"] = both
    finally:
        capi.check(lib.rt_uvm_stop(), "rt_uvm_stop")
        for p in ptrs:
            lib.rt_uvm_unregister_ptr(p)
            cudart.cudaFree(p)
    return out


def feedback_leg(torch, dev, stream, steps=100, warm=8, cpu=True):
    """The event-driven path on the incremental decode trace (65,536-slot pool,
    40 layers, Poisson arrivals, one token per live request per step):
    rt_feedback_step (allocation event + attention event + plan in one launch) with
    every index tensor already in HBM, launched step by step and as one captured
    graph, and the same steps as the three separate calls; beside it the Python restatement of
    SlotFeedback.consume -> publish -> target_blocks -> choose -> blocksv on one core."""
    from retarget_b200 import capi, workloads
    from retarget_b200.feedback import DeviceFeedback
    from retarget_b200.planner import DevicePlanner, result_from_tensor
    layout = workloads.Layout(40, 2048, 65536)
    trace = workloads.decode_trace(0, steps=warm + steps, initial_requests=48)
    budget, max_blocks, active, refresh = 16, 16, 2.0, 10.0
    times = [100.0 + 0.03 * i for i in range(len(trace))]
    out = {}
    cpu_ranges = None
    if cpu:
        from oracle import compose
        from oracle import ref_policy as rp
        spec = rp.SlotSpec(block_tokens=layout.block_tokens, max_blocks_per_update=max_blocks,
                           active_seconds=active, refresh_seconds=refresh)
        session = compose.FeedbackSession(layout, spec, budget, evict=True)
        cpu_ranges, t_cpu = 0, 0.0
        for i, ev in enumerate(trace):
            t0 = time.perf_counter()
            if len(ev.alloc_slots):
                session.alloc(ev.alloc_slots, ev.free_head, times[i] - 0.002)
            session.attention(ev.read_slots, ev.write_slots, times[i])
            got, _ = session.plan(times[i] + 0.001)
            if i >= warm:
                t_cpu += time.perf_counter() - t0
                cpu_ranges += len(got)
        out["cpu_us_per_step"] = t_cpu / steps * 1e6
        out["cpu"] = "Python restatement of the reference's event-driven chain, 1 core, all timed steps"
    planner = DevicePlanner(layout, dev.index or 0)
    fb = DeviceFeedback(planner, pid=0)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    d_steps = [(up(ev.alloc_slots) if len(ev.alloc_slots) else None,
                up(ev.free_head) if ev.free_head is not None and len(ev.alloc_slots) else None,
                up(ev.read_slots), up(ev.write_slots)) for ev in trace]
    d_out = torch.zeros((1 << 14) * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    h = stream.cuda_stream

    policy = dict(budget=budget, max_blocks_per_update=max_blocks, active_seconds=active, refresh_seconds=refresh,
                  flags=capi.RT_PLAN_EVICT, d_out=d_out, d_result=d_res, stream=h)

    def three_calls(i):
        a, head, r, w = d_steps[i]
        if a is not None:
            fb.alloc(a, times[i] - 0.002, head, h)
        fb.attention(r, w, times[i], h)
        fb.plan(times[i] + 0.001, **policy)

    def one_launch(i):
        a, head, r, w = d_steps[i]
        fb.step(d_allocated=a, t_allocated=times[i] - 0.002, d_free_head=head, d_read=r, d_written=w,
                t_attention=times[i], now=times[i] + 0.001, **policy)

    def restart():
        fb.clear(99.0, h)
        planner.set_resident([set()])

    def timed(step, graph=False):
        """The trace from the start: `warm` untimed steps, then `steps` timed ones --
        launched one by one, or (graph) captured once and replayed as one graph."""
        restart()
        for i in range(warm):
            step(i)
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(warm, warm + steps):
                    step(i)
            ev[0].record(stream)
            g.replay()
        else:
            ev[0].record(stream)
            for i in range(warm, warm + steps):
                step(i)
        ev[1].record(stream)
        torch.cuda.synchronize()
        return ev[0].elapsed_time(ev[1]) * 1e3 / steps

    out["three_calls_us_per_step"] = timed(three_calls)
    out["one_launch_us_per_step"] = timed(one_launch)
    out["one_launch_graph_us_per_step"] = timed(one_launch, graph=True)
    out["us_per_step"] = out["one_launch_us_per_step"]
    # the same trace again, one step at a time, to count the ranges
    restart()
    gpu_ranges = 0
    for i in range(warm + steps):
        one_launch(i)
        stream.synchronize()
        if i >= warm:
            gpu_ranges += result_from_tensor(d_res)["n_ranges"]
    ids = sum(len(e.alloc_slots) + len(e.read_slots) + len(e.write_slots) for e in trace[warm:]) / steps
    out.update(steps=steps, event_ids_per_step=ids, launches_per_step=1,
               three_calls_launches_per_step=sum(2 + (a is not None) for a, *_ in d_steps[warm:]) / steps,
               ranges_total=gpu_ranges, workload="incremental decode trace L40 S65536, event-driven feedback state")
    if cpu_ranges is not None:
        out["ranges_match_cpu"] = cpu_ranges == gpu_ranges
    fb.close()
    planner.close()
    return out


# DRAM bytes per launch of the scan kernel from the ncu captures summarised under
# profiles/ (dram__bytes_read.sum + dram__bytes_write.sum, mean of 3 launches), keyed by
# (workload, tma); a configuration that was not captured reports null.
PROFILED_TRAFFIC_BYTES = {
    ("target", False): 182_136_000,   # 178.34 MB read + 3.79 MB written
    ("target", True): 183_182_000,    # 178.34 MB read + 4.85 MB written
}


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def run_ours(args):
    import torch
    from retarget_b200.multirank import Ranks
    from retarget_b200 import capi, workloads
    from retarget_b200.planner import DevicePlanner

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    single = world == 1
    batches = make_batches(args.workload)
    lay = batches[0].layout
    # CPU baselines first: their worker processes are forked before CUDA is initialised
    cpu_lines = {}
    if rank == 0 and single and not args.no_cpu:
        c_s, c_threads = cpu_c_port(batches, 5)
        cpu_lines["cpu_baseline"] = {
            "value": c_s * 1e6, "unit": UNIT, "cores": c_threads, "kind": "port",
            "sample": "full step (all layers), C restatement of the reference chain with OpenMP over layers, "
                      "median of 5 steps"}
        sample = 2
        py = cpu_python_port(batches, list(range(sample)), 1, 2, 1)
        cpu_lines["cpu_baseline_python"] = {
            "value": statistics.mean(py) * 1e6, "unit": "us per step for the sampled layers", "cores": 1,
            "kind": "port", "layers_in_sample": sample, "layers_per_step": lay.n_groups,
            "sample": f"{sample} of {lay.n_groups} layers per step through the Python restatement of the "
                      f"reference chain, 1 process (the reference arm times all layers)"}
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; retarget_b200 has no CPU path to fall back to")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # RETARGET_RANKS=file: rendezvous through files, no process group (a diagnostic)
    ranks = Ranks(os.environ.get("RETARGET_RANKS", "nccl")).start(dev)
    base = capi.RT_PLAN_EVICT | (capi.RT_PLAN_TMA if args.tma else 0)
    # back-to-back steps of one plan: each may scan under the tail of the one before
    flags = base | (0 if args.unchained else capi.RT_PLAN_CHAINED)
    planner = DevicePlanner(lay, local, max_indices=max(b.n_idx for b in batches) + 8, max_ranges=1 << 16)
    d_slots = upload(torch, dev, batches)
    h_slots = [torch.from_numpy(b.slots).pin_memory() for b in batches]
    d_out = torch.zeros((1 << 16) * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    # a stream of our own: handle 0 would select the planner's internal stream
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    K, W = args.steps, args.warmup
    timer = StepTimer(torch, planner, stream, d_out, d_res, flags)

    def barrier():
        ranks.barrier()
        torch.cuda.synchronize()

    # clocks are sampled from the warm-up to the end of the end-to-end loop
    sampler = ClockSampler(local) if rank == 0 else None

    # ---- headline: device time per step ----
    n_timed, run, graph = timer.timed(d_slots, batches, min_steps=K, launch=args.launch, warm=W,
                                      min_ms=args.min_timed_ms)
    n_timed = int(ranks.max_over_ranks([n_timed])[0])       # every rank times the same number of steps
    barrier()
    total_ms = run(n_timed)
    barrier()
    n_ranges = timer.result()["n_ranges"]

    # ---- config 4 on every rank: one tensor-parallel shard per GPU ----
    tp_pair = [workloads.tp_shard(0), workloads.tp_shard(1)]
    tp_planner = DevicePlanner(tp_pair[0].layout, local)
    tp_timer = StepTimer(torch, tp_planner, stream, d_out, d_res, flags)
    tp_slots = upload(torch, dev, tp_pair)
    tp_n, tp_run, _ = tp_timer.timed(tp_slots, tp_pair, min_steps=200 if args.min_timed_ms else 20,
                                     launch=args.launch, min_ms=min(20.0, args.min_timed_ms))
    tp_n = int(ranks.max_over_ranks([tp_n])[0])
    barrier()
    tp_ms = tp_run(tp_n)
    barrier()
    tp_ranges = tp_timer.result()["n_ranges"]

    extras = {}
    if rank == 0 and single and not args.no_extras:
        try:
            def leg(pair, tensors, *, launch=args.launch, f=None, id_bytes=8, min_ms=20.0, p=None):
                t = timer if p is None else StepTimer(torch, p, stream, d_out, d_res, flags)
                n, go, _ = t.timed(tensors, pair, min_steps=50, launch=launch, min_ms=min_ms, flags=f)
                ms = go(n)
                nr = t.result()["n_ranges"]
                us = ms * 1e3 / n
                gbs = algorithmic_bytes(pair[0], nr, id_bytes) / us / 1e3
                return {"us_per_step": us, "ranges_per_step": nr, "steps": n, "gbs": gbs}

            # per-launch kernel durations: an event pair around every launch, fully serialised launches
            dur = []
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(200)]
            for i, (a, b) in enumerate(evs):
                a.record(stream)
                timer.step(d_slots, batches, i, flags=base)
                b.record(stream)
            torch.cuda.synchronize()
            dur = sorted(a.elapsed_time(b) * 1e3 for a, b in evs)
            extras["per_launch_us"] = {"launches": len(dur), "min": dur[0], "median": dur[len(dur) // 2],
                                       "p95": dur[int(len(dur) * 0.95)],
                                       "how": "one CUDA event pair around every launch, launches not chained"}
            variants = {}
            if args.workload == "target":
                variants["stream_launches"] = leg(batches, d_slots, launch="stream")
                variants["unchained_graph"] = leg(batches, d_slots, f=base)
                for kind in ("steady", "fragmented"):
                    pair = workloads.target_pair(kind)
                    tensors = upload(torch, dev, pair)
                    variants[kind] = leg(pair, tensors)
                    del tensors
                tensors = upload(torch, dev, batches, np.int32)
                variants["int32_ids"] = leg(batches, tensors, id_bytes=4)
                del tensors
                if not args.tma:
                    variants["tma_staging"] = leg(batches, d_slots, f=flags | capi.RT_PLAN_TMA)
                # the padded-table entry point (the serving engine's req_to_token layout) on the same ids:
                # one row per (layer, request), one bitmap for all buffers
                rows = batches[0].n_idx // 2176
                if rows * 2176 == batches[0].n_idx:
                    shared = dataclasses.replace(lay, shared_bitmap=True)
                    for name, dtype, width in (("table_int32_one_bitmap", np.int32, 4), ("table_int64_one_bitmap", np.int64, 8)):
                        tp = DevicePlanner(shared, local)
                        tables = [torch.from_numpy(b.slots.astype(dtype).reshape(rows, 2176)).to(dev) for b in batches]
                        lens = torch.full((rows,), 2176, dtype=torch.int32, device=dev)

                        def table_step(i, handle):
                            tp.step_table(tables[i % 2], lens, batches[0].budget_blocks, flags, d_out, d_res, handle)
                        for i in range(4):
                            table_step(i, stream.cuda_stream)
                        torch.cuda.synchronize()
                        g = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                            for i in range(100):
                                table_step(i, torch.cuda.current_stream().cuda_stream)
                        g.replay()
                        torch.cuda.synchronize()
                        n = 1000
                        t = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                        t[0].record(stream)
                        for _ in range(n // 100):
                            g.replay()
                        t[1].record(stream)
                        torch.cuda.synchronize()
                        us = t[0].elapsed_time(t[1]) * 1e3 / n
                        del g
                        variants[name] = {"us_per_step": us, "rows": rows, "stride": 2176, "steps": n,
                                          "ranges_per_step": timer.result()["n_ranges"],
                                          "gbs": width * batches[0].n_idx / us / 1e3}
                        tp.close()
                        del tables
                # the allocation-free scan (scratch in a static device array, scan only, 64-bit ids)
                fn = capi.lib.rt_scan_slots_static
                fn.restype = C.c_int
                fn.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint32, C.c_uint32, C.c_void_p,
                               C.c_void_p, C.c_void_p]
                d_bits = torch.zeros(lay.n_groups * 32, dtype=torch.int32, device=dev)

                def static_scan(i):
                    b = batches[i % 2]
                    capi.check(fn(d_slots[i % 2].data_ptr(), b.group_off.ctypes.data, lay.n_groups, lay.capacity,
                                  lay.block_tokens, lay.n_blocks, d_bits.data_ptr(), d_res.data_ptr(),
                                  stream.cuda_stream), "rt_scan_slots_static")
                for i in range(4):
                    static_scan(i)
                torch.cuda.synchronize()
                t = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                t[0].record(stream)
                for i in range(200):
                    static_scan(i)
                t[1].record(stream)
                torch.cuda.synchronize()
                us = t[0].elapsed_time(t[1]) * 1e3 / 200
                variants["static_scan_only"] = {"us_per_step": us, "steps": 200, "gbs": 8 * batches[0].n_idx / us / 1e3,
                                                "note": "rt_scan_slots_static: a memset of its scratch + one launch per call"}
                # what a pure read of the same bytes reaches (same access pattern, nothing done with the ids)
                probe = capi.lib.rt_read_probe
                probe.restype = C.c_int
                probe.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]
                d_sink = torch.zeros(1, dtype=torch.int64, device=dev)
                nbytes = 8 * batches[0].n_idx // 16 * 16

                def read_only(i, handle):
                    capi.check(probe(d_slots[i % 2].data_ptr(), nbytes, d_sink.data_ptr(), handle), "rt_read_probe")
                for i in range(4):
                    read_only(i, stream.cuda_stream)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                    for i in range(100):
                        read_only(i, torch.cuda.current_stream().cuda_stream)
                g.replay()
                torch.cuda.synchronize()
                t = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                t[0].record(stream)
                for _ in range(10):
                    g.replay()
                t[1].record(stream)
                torch.cuda.synchronize()
                us = t[0].elapsed_time(t[1]) * 1e3 / 1000
                variants["read_only_probe"] = {"us_per_step": us, "steps": 1000, "gbs": nbytes / us / 1e3,
                                               "note": "rt_read_probe over the same two id arrays, graph replays of launches "
                                                       "that overlap each other: the same bytes read and thrown away"}
                del g
                for i in range(2):      # leave the resident state as the main workload left it
                    timer.step(d_slots, batches, W + n_timed + i)
                torch.cuda.synchronize()
            extras["variants"] = variants
            # the other stated configurations
            configs = {}
            for name in ("full_refresh", "sparse"):
                pair = [make_workload(name, 0), make_workload(name, 1)]
                p = DevicePlanner(pair[0].layout, local)
                tensors = upload(torch, dev, pair)
                configs[name] = leg(pair, tensors, p=p)
                configs[name]["slot_ids_per_step"] = pair[0].n_idx
                p.close()
                del tensors
            extras["configs"] = configs
            extras["feedback"] = feedback_leg(torch, dev, stream, cpu=not args.no_cpu)
            try:
                extras["prefetch"] = prefetch_leg(torch, dev)
            except Exception as exc:                        # the headline must not die with a side measurement
                extras["prefetch"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
        except Exception as exc:                    # the headline must not die with a side measurement
            extras["extras_error"] = f"{type(exc).__name__}: {exc}"

    # ---- end to end through the host-buffer call: pinned ids -> device -> plan -> ranges on the host ----
    out_host = np.empty(1 << 16, dtype=capi.RANGE_DTYPE)

    def host_loop(tensors, steps, f=base):
        last = 0
        for i in range(2):
            planner.step_host(tensors[i % 2].numpy(), batches[i % 2].group_off, batches[i % 2].budget_blocks,
                              f, out=out_host)
        barrier()
        t0 = time.perf_counter()
        for i in range(steps):
            b = batches[i % 2]
            _, res = planner.step_host(tensors[i % 2].numpy(), b.group_off, b.budget_blocks, f, out=out_host)
            last = res.n_ranges
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / steps, last

    # the call as a user makes it: 64-bit ids in pinned host memory; the library narrows them to 32 bits
    # on the host cores and overlaps that with the copy
    e2e_s, e2e_ranges = host_loop(h_slots, max(K, 10))
    plan = out_host[:e2e_ranges].copy()      # the last timed plan, compared across ranks below
    pack_threads = planner.narrow_threads()
    narrowed = pack_threads > 0 and lay.capacity < 0x7fffffff and batches[0].n_idx >= 1 << 20 and not args.tma
    # the same call told to copy the 64-bit ids as they are
    e2e_wide_s, wide_ranges = host_loop(h_slots, max(K, 10), base | capi.RT_PLAN_WIDE_COPY)
    if wide_ranges != e2e_ranges or not np.array_equal(out_host[:wide_ranges], plan):
        raise SystemExit("bench.py: the narrowed and the wide host-buffer calls disagree")
    # the same call on the engine's own 32-bit ids: half the bytes over the host link
    h32 = [torch.from_numpy(b.slots.astype(np.int32)).pin_memory() for b in batches]
    e2e32_s, _ = host_loop(h32, max(K, 10))
    del h32
    # ceiling of the host-buffer call: every rank doing nothing but its pinned copy
    stage = torch.empty_like(d_slots[0])
    for i in range(2):
        stage.copy_(h_slots[i], non_blocking=True)
    barrier()
    t0 = time.perf_counter()
    n_copy = 10
    for i in range(n_copy):
        stage.copy_(h_slots[i % 2], non_blocking=True)
    torch.cuda.synchronize()
    copy_s = (time.perf_counter() - t0) / n_copy
    del stage
    host_loop(h_slots, 2)                    # back to the main pair's resident state
    clocks = sampler.stop() if sampler else None

    ms_per_step, tp_ms_per_step, e2e_ms, e2e32_ms, copy_ms, e2e_wide_ms = ranks.max_over_ranks(
        [total_ms / n_timed, tp_ms / tp_n, e2e_s * 1e3, e2e32_s * 1e3, copy_s * 1e3, e2e_wide_s * 1e3])
    # every rank planned from the same slot table: the plans must agree
    # (dst names the rank's own GPU; the rest must agree)
    plans_agree = ranks.same_everywhere(b"".join(plan[k].tobytes() for k in ("buffer", "offset", "bytes")))

    if rank == 0:
        peaks_path = ROOT / "MEASURED_PEAKS.json"
        if peaks_path.exists():
            peak, peak_src = float(json.loads(peaks_path.read_text())["hbm_gbs"]), "measured"
        else:
            peak, peak_src = FALLBACK_HBM_GBS, "fallback"
        bytes_step = algorithmic_bytes(batches[0], n_ranges)
        achieved = bytes_step / (ms_per_step * 1e-3) / 1e9
        tp_bytes = algorithmic_bytes(tp_pair[0], tp_ranges)
        line = {
            "metric": METRIC, "value": ms_per_step * 1e3, "unit": UNIT, "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
            "config": workload_config(batches[0], args),
            "timed_steps": n_timed, "timed_region_ms": ms_per_step * n_timed,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "traffic": PROFILED_TRAFFIC_BYTES.get((args.workload, bool(args.tma))),
                         "peak_source": peak_src, "algorithmic_bytes_per_launch": bytes_step,
                         "launch_ms": ms_per_step,
                         "kernel": "scan_plan_tma_kernel" if args.tma else "scan_plan_kernel"},
            "e2e": {"value": e2e_ms * 1e3, "unit": UNIT,
                    "h2d_bytes_per_step": (4 if narrowed else 8) * batches[0].n_idx,
                    "d2h_bytes_per_step": 24 * e2e_ranges + 64,
                    "host_id_bytes_per_step": 8 * batches[0].n_idx,
                    "how": (f"rt_plan_step on 64-bit ids in pinned host memory: narrowed to 32 bits by {pack_threads} "
                            "host threads in chunks of 2^21 ids, every chunk's copy overlapping the next chunk's "
                            "narrowing" if narrowed else
                            "rt_plan_step on 64-bit ids in pinned host memory, copied as they are (too few host "
                            "CPUs per GPU for narrowing to pay)"),
                    "host_pack_threads": pack_threads if narrowed else 0,
                    "wide_copy_us": e2e_wide_ms * 1e3, "wide_h2d_bytes_per_step": 8 * batches[0].n_idx,
                    "int32_ids_us": e2e32_ms * 1e3, "int32_h2d_bytes_per_step": 4 * batches[0].n_idx,
                    "h2d_copy_only_us": copy_ms * 1e3,
                    "frac_of_h2d_ceiling": copy_ms / e2e_wide_ms,
                    "limiter": "the pinned host -> device copy of the slot ids (PCIe and, with several "
                               "ranks, the one host NUMA node all GPUs copy from); wide_copy_us is the call "
                               "that copies all 8 bytes per id, h2d_copy_only_us that copy alone, "
                               "int32_ids_us the call on ids the caller already holds as 32-bit"},
            "gpu_launches": n_timed,
            "clocks": clocks,
            "slot_scan_gbs_aggregate": world * achieved,
            "plans_per_s_aggregate": world / (ms_per_step * 1e-3),
            "ranges_per_step": n_ranges,
            "plans_agree_across_ranks": plans_agree,
            "tp_shard_us": tp_ms_per_step * 1e3,
            "tp_shard": {"us_per_step": tp_ms_per_step * 1e3, "steps": tp_n, "ranges_per_step": tp_ranges,
                         "slot_ids_per_step": tp_pair[0].n_idx,
                         "gbs": tp_bytes / (tp_ms_per_step * 1e-3) / 1e9,
                         "frac": tp_bytes / (tp_ms_per_step * 1e-3) / 1e9 / peak,
                         "workload": "48 layers, one KV head per rank (256 B slots), 262,144-slot pool, "
                                     "256 requests; every rank plans its own shard"},
        }
        for name, cfg in extras.get("configs", {}).items():
            cfg["frac"] = cfg["gbs"] / peak
        line.update(extras)
        line.update(cpu_lines)
        emit(line)
    tp_planner.close()
    planner.close()
    ranks.stop()


# --------------------------------------------------------------------------
# event-driven path alone
# --------------------------------------------------------------------------
def run_feedback(args):
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; retarget_b200 has no CPU path to fall back to")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    sampler = ClockSampler(0)
    got = feedback_leg(torch, dev, stream, steps=args.steps, warm=max(args.warmup, 3), cpu=not args.no_cpu)
    line = {"metric": "feedback_plan_us_per_decode_step", "value": got["us_per_step"], "unit": UNIT, "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": got["us_per_step"] / 1e3,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "int64",
            "data": "synthetic", "config": {"workload": got["workload"]}, "feedback": got,
            "clocks": sampler.stop()}
    emit(line)


# --------------------------------------------------------------------------
# end to end: plan -> prefetch -> paged decode attention, every decode step
# --------------------------------------------------------------------------
def run_e2e_prefetch(args):
    """--workload e2e_prefetch: the oversubscribed end-to-end configuration at the
    largest size that is safe on a shared host.

    K and V of every layer live in managed memory registered with the in-process
    UVM server; a managed ballast (co-resident training tensors) is touched every
    step.  An incremental decode trace runs for `--steps` steps.  Each step, arm
    by arm:

      plan         the device planner turns THAT step's slot table into ranges
                   (evictions first), rt_uvm_submit_ranges hands them to the
                   executor on its side streams, then the attention reader runs
      plan_ahead   the same plan one step ahead: while the reader of step i runs
                   on the main stream, the executor brings in what step i+1 adds
                   on its side streams; what step i+1 evicts is moved out only
                   after the reader of step i has finished (it may still be
                   reading those blocks)
      no_prefetch  the same evictions are executed (same residency pressure) but
                   nothing is brought in ahead: the reader's first touch of a new
                   block faults it in
      resident     everything on the GPU, no plan: the floor of the reader

    The footprint is scaled down (the full 160 GiB + 20 GiB would need as much
    host memory again on a machine shared with other jobs): a GPU share limit is
    emulated by the plan's own evictions instead of by real oversubscription, and
    pages are handed out in address order so that the live set is a region a
    bounded plan can follow.  UVM fault counts: unavailable (CUPTI's
    unified-memory counters cannot be enabled with this toolkit and driver)."""
    import torch
    from cuda.bindings import driver as cu
    from cuda.bindings import runtime as cudart
    from retarget_b200 import capi, workloads
    from retarget_b200.control import LocalUvm
    from retarget_b200.planner import DevicePlanner, ranges_from_tensor, result_from_tensor

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; retarget_b200 has no CPU path to fall back to")
    K, W = max(args.steps, 64), max(args.warmup, 3)
    lib = capi.lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    torch.zeros(1, device=dev)
    err, concurrent = cudart.cudaDeviceGetAttribute(cudart.cudaDeviceAttr.cudaDevAttrConcurrentManagedAccess, 0)
    if int(err) != 0 or not concurrent:
        emit({"metric": "e2e_decode_step_ms", "unavailable": "device has no concurrent managed access"})
        return
    # ---- sizes: at most a quarter of the host memory that is available right now ----
    layers, heads, bytes_per_slot = 40, 8, 2048
    avail = 0
    for text in Path("/proc/meminfo").read_text().splitlines():
        if text.startswith("MemAvailable:"):
            avail = int(text.split()[1]) * 1024
    pool_slots = 131072                                       # 256 MiB per buffer, 20 GiB of K + V
    while pool_slots > 8192 and 2 * layers * pool_slots * bytes_per_slot * 1.1 > avail / 4:
        pool_slots //= 2
    alloc = pool_slots * bytes_per_slot
    total = 2 * layers * alloc
    ballast_bytes = max(64 * MIB, total // 8 // (2 * MIB) * (2 * MIB))     # 20 GiB : 160 GiB in the full configuration
    layout = workloads.Layout(layers, bytes_per_slot, pool_slots)        # one bitmap for all buffers
    budget = layout.n_blocks * 3 // 4                                    # the GPU share the plan may fill
    # requests sized so that the live set stays well inside the pool
    median = max(256, pool_slots // 96)
    trace = workloads.decode_trace(0, steps=W + K, pool_slots=pool_slots, arrival_rate=0.25, median=median,
                                   mean_output=256, initial_requests=24, shuffle_pages=False)
    err, ctx = cu.cuCtxGetCurrent()
    ptrs = []
    def release():
        for q in ptrs:
            lib.rt_uvm_unregister_ptr(q)
            cudart.cudaFree(q)
    for _ in range(2 * layers + 1):
        size = alloc if len(ptrs) < 2 * layers else ballast_bytes
        err, p = cudart.cudaMallocManaged(size, cudart.cudaMemAttachGlobal)
        if int(err) != 0:
            release()
            emit({"metric": "e2e_decode_step_ms", "unavailable": f"cudaMallocManaged failed: {err}"})
            return
        ptrs.append(int(p))
        cudart.cudaMemset(p, 0x3c if len(ptrs) % 2 else 0x3d, size)       # bf16 values near 0.01 / 0.05
    torch.cuda.synchronize()
    lib.rt_uvm_register.argtypes = [C.c_uint64, C.c_uint64, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_uint64)]
    lib.rt_uvm_unregister_ptr.argtypes = [C.c_uint64]
    lib.rt_uvm_submit_ranges.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.POINTER(C.c_uint64)]
    lib.rt_uvm_wait.argtypes = [C.c_uint64, C.c_double, C.POINTER(C.c_int)]
    lib.rt_paged_attention.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p]
    lib.rt_paged_read.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint64,
                                  C.c_void_p, C.c_void_p]
    ids = []
    for k, p in enumerate(ptrs):
        i = C.c_uint64()
        capi.check(lib.rt_uvm_register(p, alloc if k < 2 * layers else ballast_bytes, C.c_void_p(int(ctx)), 0, 1,
                                       C.byref(i)), "rt_uvm_register")
        ids.append(i.value)
    kv_ids = (C.c_uint64 * (2 * layers))(*ids[:2 * layers])
    uvm = LocalUvm()
    cfg = capi.UvmConfig(None, 64 * MIB, 1024 * MIB, 4, 0)
    capi.check(lib.rt_uvm_start(C.byref(cfg)), "rt_uvm_start")
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    h = stream.cuda_stream
    # yardstick for the prefetch rate
    host = torch.empty(256 * MIB, dtype=torch.uint8).pin_memory()
    devbuf = torch.empty(256 * MIB, dtype=torch.uint8, device=dev)
    devbuf.copy_(host, non_blocking=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(4):
        devbuf.copy_(host, non_blocking=True)
    torch.cuda.synchronize()
    h2d = 4 * 256 * MIB / (time.perf_counter() - t0) / 1e9
    del host, devbuf
    # device-side inputs of the reader
    max_live = max(t.live for t in trace)
    d_k = torch.tensor(ptrs[:layers], dtype=torch.int64, device=dev)             # K buffers first, then V
    d_v = torch.tensor(ptrs[layers:2 * layers], dtype=torch.int64, device=dev)
    q = (torch.randn(max_live, layers, heads, 128, device=dev) * 0.5).to(torch.bfloat16)
    out = torch.zeros(max_live, layers, heads, 128, dtype=torch.float32, device=dev)
    d_steps = [(torch.from_numpy(t.read_slots).to(dev), torch.from_numpy(t.req_off).to(dev), t.live) for t in trace]
    d_ballast = torch.tensor([ptrs[-1]], dtype=torch.int64, device=dev)
    ballast_rows = ballast_bytes // bytes_per_slot
    touch = torch.arange(1, min(ballast_rows, 32768), dtype=torch.int64, device=dev)    # 64 MiB of the ballast
    d_sum = torch.zeros(1, dtype=torch.int64, device=dev)
    d_out = torch.zeros((1 << 14) * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    planner = DevicePlanner(layout, 0)
    sampler = ClockSampler(0)

    def migrate(line):
        reply = uvm.command(line)
        assert reply.get("ok"), reply
        uvm._wait_job(reply["job_id"], timeout=600, poll_seconds=0.0005)

    def read(i):
        slots, off, live = d_steps[i]
        capi.check(lib.rt_paged_read(d_ballast.data_ptr(), 1, bytes_per_slot, touch.data_ptr(), touch.numel(),
                                     ballast_rows - 1, d_sum.data_ptr(), h), "rt_paged_read")
        capi.check(lib.rt_paged_attention(d_k.data_ptr(), d_v.data_ptr(), layers, heads, q.data_ptr(),
                                          slots.data_ptr(), off.data_ptr(), live, layout.capacity,
                                          out.data_ptr(), h), "rt_paged_attention")
        stream.synchronize()

    def arm(kind):
        gen = uvm.status().allocation_generation
        kv_total = 2 * layers * alloc
        # start: K and V on the CPU (plan / no_prefetch) or everything on the GPU (resident)
        migrate(f"targetv {gen} {kv_total + ballast_bytes if kind == 'resident' else 0}")
        if kind != "resident":
            migrate(f"prefetch {ids[-1]} 0 {ballast_bytes} gpu")
        planner.set_resident([set()])
        t_step = t_plan = t_move = t_read = 0.0
        moved = to_gpu = 0
        n_ranges = 0
        for i in range(W + K):
            slots, off, live = d_steps[i]
            a = time.perf_counter()
            b = c = a
            if kind != "resident":
                planner.step_device(slots, np.array([0, slots.numel()], np.int64), budget, capi.RT_PLAN_EVICT,
                                    d_out, d_res, h)
                stream.synchronize()
                res = result_from_tensor(d_res)
                if res["flags"]:
                    raise SystemExit(f"bench.py: planner reported flags {res['flags']}")
                ranges = ranges_from_tensor(d_out, res["n_ranges"])
                if kind == "no_prefetch":
                    ranges = ranges[:res["n_cpu_ranges"]]           # the evictions only
                b = time.perf_counter()
                if len(ranges):
                    job, cuda_err = C.c_uint64(), C.c_int()
                    keep = np.ascontiguousarray(ranges)
                    capi.check(lib.rt_uvm_submit_ranges(keep.ctypes.data, len(keep), kv_ids, 2 * layers,
                                                        C.byref(job)), "rt_uvm_submit_ranges")
                    capi.check(lib.rt_uvm_wait(job.value, 600.0, C.byref(cuda_err)), "rt_uvm_wait")
                    if cuda_err.value:
                        raise SystemExit(f"bench.py: prefetch job failed with CUDA error {cuda_err.value}")
                c = time.perf_counter()
            read(i)
            d = time.perf_counter()
            if i >= W:
                t_step += d - a; t_plan += b - a; t_move += c - b; t_read += d - c
                if kind != "resident":
                    n_ranges += len(ranges)
                    moved += int(ranges["bytes"].sum())
                    to_gpu += int(ranges["bytes"][ranges["dst"] >= 0].sum())
        rec = {"step_ms": t_step / K * 1e3, "plan_ms": t_plan / K * 1e3, "prefetch_ms": t_move / K * 1e3,
               "reader_ms": t_read / K * 1e3, "ranges_per_step": n_ranges / K,
               "bytes_moved_per_step": moved / K, "bytes_to_gpu_per_step": to_gpu / K}
        if kind == "plan" and t_move > 0:
            rec["prefetch_gbs_while_moving"] = moved / t_move / 1e9
            rec["prefetch_frac_of_link"] = moved / t_move / 1e9 / h2d
        return rec

    def submit(ranges):
        if not len(ranges):
            return None
        job = C.c_uint64()
        keep = np.ascontiguousarray(ranges)
        capi.check(lib.rt_uvm_submit_ranges(keep.ctypes.data, len(keep), kv_ids, 2 * layers, C.byref(job)),
                   "rt_uvm_submit_ranges")
        return job.value

    def wait(job):
        if job is None:
            return
        cuda_err = C.c_int()
        capi.check(lib.rt_uvm_wait(job, 600.0, C.byref(cuda_err)), "rt_uvm_wait")
        if cuda_err.value:
            raise SystemExit(f"bench.py: prefetch job failed with CUDA error {cuda_err.value}")

    def plan_of(i):
        slots, off, live = d_steps[i]
        planner.step_device(slots, np.array([0, slots.numel()], np.int64), budget, capi.RT_PLAN_EVICT,
                            d_out, d_res, h)
        stream.synchronize()
        res = result_from_tensor(d_res)
        if res["flags"]:
            raise SystemExit(f"bench.py: planner reported flags {res['flags']}")
        ranges = ranges_from_tensor(d_out, res["n_ranges"])
        return ranges[:res["n_cpu_ranges"]], ranges[res["n_cpu_ranges"]:]

    def arm_ahead():
        gen = uvm.status().allocation_generation
        migrate(f"targetv {gen} 0")
        migrate(f"prefetch {ids[-1]} 0 {ballast_bytes} gpu")
        planner.set_resident([set()])
        evict, add = plan_of(0)
        wait(submit(add))                                   # the first step's blocks, before the loop
        t_step = t_read = 0.0
        moved = 0
        for i in range(W + K):
            a = time.perf_counter()
            if i + 1 < W + K:
                evict, add = plan_of(i + 1)                 # next step's table: known once the step is scheduled
                job = submit(add)                           # moves in under the reader, on the side streams
            else:
                evict, add, job = evict[:0], add[:0], None
            b = time.perf_counter()
            read(i)
            c = time.perf_counter()
            wait(job)
            wait(submit(evict))                             # only now: the reader of step i is done with them
            d = time.perf_counter()
            if i >= W:
                t_step += d - a; t_read += c - b
                moved += int(add["bytes"].sum()) + int(evict["bytes"].sum())
        return {"step_ms": t_step / K * 1e3, "reader_ms": t_read / K * 1e3, "bytes_moved_per_step": moved / K}

    try:
        arms = {kind: arm(kind) for kind in ("resident", "no_prefetch", "plan")}
        arms["plan_ahead"] = arm_ahead()
    finally:
        capi.check(lib.rt_uvm_stop(), "rt_uvm_stop")
        planner.close()
        release()
    live_slots = statistics.mean(int(s.numel()) for s, _, _ in d_steps[W:])
    line = {"metric": "e2e_decode_step_ms", "value": arms["plan_ahead"]["step_ms"], "unit": "ms/step", "n_gpus": 1,
            "steps": K, "warmup": W, "ms_per_step": arms["plan_ahead"]["step_ms"], "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 rows, fp32 accumulate (reader); int64 ids (plan)",
            "data": "synthetic",
            "config": {"workload": "incremental decode trace over managed K/V: plan -> prefetch -> paged decode "
                                   "attention, every step", "layers": layers, "kv_buffers": 2 * layers,
                       "alloc_bytes": alloc, "kv_bytes_total": total, "ballast_bytes": ballast_bytes,
                       "pool_slots": pool_slots, "blocks_per_bitmap": layout.n_blocks, "budget_blocks": budget,
                       "live_slots_mean": live_slots, "live_requests_max": max_live,
                       "reader_bytes_per_step": live_slots * 2 * layers * bytes_per_slot,
                       "host_memory_available_bytes": avail,
                       "host_memory_margin": "K + V + ballast sized to at most a quarter of MemAvailable",
                       "page_order": "address order (the live set is a moving region)"},
            "arms": arms, "h2d_link_gbs": h2d,
            "um_fault_counts": "unavailable: CUPTI's unified-memory counter activity cannot be enabled with this "
                               "toolkit and driver",
            "clocks": sampler.stop()}
    emit(line)


# Libraries under us (NCCL's version banner, for one) write to stdout.  The
# result line must be the only thing there: everything else goes to stderr.
_RESULT_FD = None


def quiet_stdout():
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict):
    text = json.dumps(line) + "\n"
    if _RESULT_FD is None:
        sys.stdout.write(text)
        sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_RESULT_FD, text.encode())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed steps (default 200; 20 for --impl reference, whose steps take a second each)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="target",
                    choices=["target", "steady", "fragmented", "sparse", "full_refresh", "tp_shard", "feedback",
                             "e2e_prefetch"])
    ap.add_argument("--tma", action="store_true", help="stage ids with bulk async copies (TMA)")
    ap.add_argument("--launch", default="graph", choices=["graph", "stream"],
                    help="how the timed launches are issued: CUDA graph replays or one by one")
    ap.add_argument("--unchained", action="store_true",
                    help="launch every step fully serialised after the one before it (no RT_PLAN_CHAINED)")
    ap.add_argument("--min-timed-ms", type=float, default=MIN_TIMED_MS,
                    help="shortest timed region of the headline figure; 0 times exactly --steps steps "
                         "(profiling runs)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--no-extras", "--no-variants", dest="no_extras", action="store_true",
                    help="skip the secondary measurements (variants, configs, feedback, prefetch)")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = 20 if args.impl == "reference" else 200
    if args.impl == "ours":
        args.warmup = max(args.warmup, 3)
        args.steps = max(args.steps, 2)
    quiet_stdout()
    if args.workload == "feedback":
        run_feedback(args)
    elif args.workload == "e2e_prefetch":
        run_e2e_prefetch(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
