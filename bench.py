#!/usr/bin/env python3
"""Placement-plan benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
                    [--launch graph|stream] [--tma] [--no-cpu] [--no-variants]

One step = one placement plan for one decode step of the headline workload:
40 layers (80 KV buffers of 512 MiB), 256 requests, a 262,144-slot pool, and per
(layer, request) touched sets of the newest 128 slots plus 2048 Zipf(1.1)
history draws -- 22.3 M int64 slot ids (178 MB) per step.  Two different
batches alternate, so every step re-reads more than the L2 holds; one lives in
the lower half of every buffer and one in the upper half, so every plan evicts
one run and adds one run per buffer (160 ranges per step, the shape of the
reference's incremental window update).  `variants` reports the same step when
nothing moves (0 ranges), when the whole budget is replaced in single-block
runs (6080 ranges) and when the ids are int32.

`value`  device time per step, slot ids already in HBM (two CUDA events on the
         launching stream around the K steps, max over ranks); the steps are
         issued as CUDA-graph replays (--launch graph, default) or one by one
--workload feedback  the event-driven path (device-resident feedback state)
         on an incremental decode trace, beside the Python chain on one core
`e2e`    the same plan through the host-buffer C-ABI call: pinned host ids are
         copied to the device, planned, and the range list is copied back
--impl reference  times the CPU restatement of the reference's Python path on
         the host cores (a bounded sample of layers per step, scaled up)

Prints one JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
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


def algorithmic_bytes(batch, n_ranges: int) -> int:
    """Bytes one step must move: every slot id once, the group offsets, the
    resident words read and written, the ranges and the result record."""
    G = batch.layout.n_groups
    return 8 * batch.n_idx + 8 * (G + 1) + 2 * 4 * 32 * G + 24 * n_ranges + 64


def workload_config(batch, extra=None) -> dict:
    lay = batch.layout
    name = batch.name
    for tag, text in ((", lower half", ", steps alternate between the lower and upper half of every buffer"),
                      (", even blocks", ", steps alternate between even and odd blocks")):
        if name.endswith(tag):
            name = name[:-len(tag)] + text
    cfg = {"workload": name, "layers": lay.layers, "kv_buffers": lay.n_buffers,
           "alloc_bytes": lay.alloc_bytes, "pool_slots": lay.pool_slots,
           "bytes_per_slot": lay.bytes_per_slot, "uvm_block_bytes": lay.block_bytes,
           "bitmaps": lay.n_groups, "blocks_per_bitmap": lay.n_blocks,
           "budget_blocks": batch.budget_blocks, "slot_ids_per_step": batch.n_idx,
           "slot_id_bytes_per_step": 8 * batch.n_idx, "index_dtype": "int64"}
    cfg.update(extra or {})
    return cfg


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
    import dataclasses
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


def cpu_python_port(batches, sample_layers: int, procs: int, steps: int, warmup: int):
    """Times the Python restatement of the reference path on `sample_layers`
    layers per step (spread over `procs` processes) and scales to all layers.
    Returns per-step seconds for the whole workload."""
    L = batches[0].layout.n_groups
    _CPU["batches"] = batches
    resident = {}
    layers = list(range(min(sample_layers, L)))
    ctx = mp.get_context("fork")
    times = []
    with ctx.Pool(procs) as pool:
        for step in range(warmup + steps):
            t = time.perf_counter()
            res = pool.map(_cpu_layer, [(step % 2, l, resident.get(l, ())) for l in layers],
                           chunksize=1)
            dt = time.perf_counter() - t
            for _, _, layer, blocks in res:
                resident[layer] = blocks
            if step >= warmup:
                times.append(dt * L / len(layers))
    return times


def cpu_c_port(batches, reps: int):
    from oracle import c_oracle
    co = c_oracle.COracle(batches[0].layout)
    threads = min(co.max_threads, os.cpu_count() or 1)
    times = []
    for i in range(reps + 1):
        b = batches[i % 2]
        t = time.perf_counter()
        co.step(b.slots, b.group_off, b.budget_blocks, True, threads)
        if i:
            times.append(time.perf_counter() - t)
    return statistics.median(times), threads


def run_reference(args):
    """The reference arm: CPU only, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    batches = make_batches(args.workload)
    cores = os.cpu_count() or 1
    L = batches[0].layout.n_groups
    sample = min(L, max(1, cores))
    times = cpu_python_port(batches, sample, min(cores, sample), args.steps, args.warmup)
    per_step = statistics.mean(times)
    us = per_step * 1e6
    sample_text = (f"{sample} of {L} layers per step through the Python restatement of "
                   f"encode_runs->blocks->target_blocks->choose->blocksv, {min(cores, sample)} "
                   f"processes, scaled x{L / sample:.2f}")
    line = {"impl": "reference", "metric": METRIC, "value": us, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "int64",
            "data": "synthetic", "config": workload_config(batches[0]),
            "cpu_baseline": {"value": us, "unit": UNIT, "cores": min(cores, sample), "kind": "port",
                             "sample": sample_text},
            "e2e": {"value": us, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def run_ours(args):
    import torch
    from retarget_b200.multirank import Ranks
    from retarget_b200 import capi
    from retarget_b200.planner import DevicePlanner, result_from_tensor

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    batches = make_batches(args.workload)
    lay = batches[0].layout
    # CPU baseline first: its worker processes are forked before CUDA is initialised
    cpu_lines = {}
    if rank == 0 and world == 1 and not args.no_cpu:
        sample = 2
        L = lay.n_groups
        py = cpu_python_port(batches, sample, 1, 2, 1)
        c_s, c_threads = cpu_c_port(batches, 3)
        cpu_lines["cpu_baseline"] = {
            "value": statistics.mean(py) * 1e6, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": f"{min(sample, L)} of {L} layers per step through the Python restatement of "
                      f"the reference chain, 1 process, scaled x{L / min(sample, L):.0f}"}
        cpu_lines["cpu_baseline_native"] = {
            "value": c_s * 1e6, "unit": UNIT, "cores": c_threads, "kind": "port",
            "sample": "full step, C restatement with OpenMP over layers"}
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; retarget_b200 has no CPU path to fall back to")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    ranks = Ranks("nccl").start(dev)
    flags = capi.RT_PLAN_EVICT | (capi.RT_PLAN_TMA if args.tma else 0)
    # back-to-back steps of one plan: each may scan under the tail of the one before
    if not args.unchained:
        flags |= capi.RT_PLAN_CHAINED
    planner = DevicePlanner(lay, local, max_indices=max(b.n_idx for b in batches) + 8,
                            max_ranges=1 << 16)
    d_slots = [torch.from_numpy(b.slots).to(dev) for b in batches]
    h_slots = [torch.from_numpy(b.slots).pin_memory() for b in batches]
    d_out = torch.zeros((1 << 16) * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    # a stream of our own: handle 0 would select the planner's internal stream
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    K, W = args.steps, args.warmup

    def barrier():
        ranks.barrier()
        torch.cuda.synchronize()

    def device_step(i):
        b = batches[i % 2]
        planner.step_device(d_slots[i % 2], b.group_off, b.budget_blocks, flags, d_out, d_res,
                            stream.cuda_stream)

    # clocks are sampled from the warm-up to the end of the end-to-end loop: the
    # device-timed region alone lasts only a few milliseconds
    sampler = ClockSampler(local) if rank == 0 else None
    for i in range(W):
        device_step(i)
    torch.cuda.synchronize()
    n_ranges = result_from_tensor(d_res)["n_ranges"]

    # The K launches go out the way a serving engine issues its decode step: as
    # nodes of a CUDA graph (--launch graph, the default; an even number of steps
    # is captured once and replayed, what does not fill a replay is launched
    # plainly) or one by one on the stream (--launch stream).  One event on either
    # side of the K launches: an event between every two launches is measurement
    # overhead on the stream (about 2.5 us each here).
    graph, per_replay = None, 0
    if args.launch == "graph" and K >= 2:
        per_replay = min(20, K - K % 2)
        graph = torch.cuda.CUDAGraph()
        # thread-local capture mode: the process group's watchdog thread may query events meanwhile
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            for i in range(per_replay):
                b = batches[(W + i) % 2]
                planner.step_device(d_slots[(W + i) % 2], b.group_off, b.budget_blocks, flags, d_out,
                                    d_res, torch.cuda.current_stream().cuda_stream)
        graph.replay()                        # untimed: first replay of a new graph
        torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    barrier()
    ev[0].record(stream)
    done = 0
    if graph is not None:
        for _ in range(K // per_replay):
            graph.replay()
        done = K // per_replay * per_replay
    for i in range(done, K):
        device_step(W + i)
    ev[1].record(stream)
    barrier()
    total_ms = ev[0].elapsed_time(ev[1])
    last = result_from_tensor(d_res)
    if last["flags"]:
        raise SystemExit(f"bench.py: planner reported flags {last['flags']}")

    # the same step under other conditions (headline workload, one GPU only)
    variants = {}
    if args.workload == "target" and world == 1 and not args.no_variants:
        def timed(slot_tensors, pair, n=50):
            def one(i):
                planner.step_device(slot_tensors[i % 2], pair[i % 2].group_off,
                                    pair[i % 2].budget_blocks, flags, d_out, d_res, stream.cuda_stream)
            for i in range(4):
                one(i)
            torch.cuda.synchronize()
            t = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            t[0].record(stream)
            for i in range(n):
                one(i)
            t[1].record(stream)
            torch.cuda.synchronize()
            r = result_from_tensor(d_res)
            if r["flags"]:
                raise SystemExit(f"bench.py: planner reported flags {r['flags']}")
            return t[0].elapsed_time(t[1]) * 1e3 / n, r["n_ranges"], n

        from retarget_b200 import workloads
        us, nr, n = timed(d_slots, batches)
        variants["stream_launches"] = {"us_per_step": us, "ranges_per_step": nr, "steps": n,
                                       "gbs": algorithmic_bytes(batches[0], nr) / us / 1e3}
        for kind in ("steady", "fragmented"):
            pair = workloads.target_pair(kind)
            tensors = [torch.from_numpy(b.slots).to(dev) for b in pair]
            us, nr, n = timed(tensors, pair)
            variants[kind] = {"us_per_step": us, "ranges_per_step": nr, "steps": n,
                              "gbs": algorithmic_bytes(pair[0], nr) / us / 1e3}
            del tensors
        tensors = [torch.from_numpy(b.slots.astype(np.int32)).to(dev) for b in batches]
        us, nr, n = timed(tensors, batches)
        variants["int32_ids"] = {"us_per_step": us, "ranges_per_step": nr, "steps": n,
                                 "gbs": (algorithmic_bytes(batches[0], nr) - 4 * batches[0].n_idx) / us / 1e3}
        del tensors
        # the padded-table entry point (the serving engine's req_to_token layout) on the same ids as
        # int32: one row per (layer, request), one bitmap for all buffers
        rows = batches[0].n_idx // 2176
        if rows * 2176 == batches[0].n_idx:
            shared = dataclasses.replace(lay, shared_bitmap=True)
            table_planner = DevicePlanner(shared, local)
            tables = [torch.from_numpy(b.slots.astype(np.int32).reshape(rows, 2176)).to(dev) for b in batches]
            lens = torch.full((rows,), 2176, dtype=torch.int32, device=dev)
            for i in range(4):
                table_planner.step_table(tables[i % 2], lens, batches[0].budget_blocks, flags, d_out, d_res,
                                         stream.cuda_stream)
            torch.cuda.synchronize()
            t = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            t[0].record(stream)
            for i in range(50):
                table_planner.step_table(tables[i % 2], lens, batches[0].budget_blocks, flags, d_out, d_res,
                                         stream.cuda_stream)
            t[1].record(stream)
            torch.cuda.synchronize()
            us = t[0].elapsed_time(t[1]) * 1e3 / 50
            variants["table_int32_one_bitmap"] = {"us_per_step": us, "rows": rows, "stride": 2176, "steps": 50,
                                                  "ranges_per_step": result_from_tensor(d_res)["n_ranges"],
                                                  "gbs": 4 * batches[0].n_idx / us / 1e3}
            table_planner.close()
            del tables
        for i in range(2):      # leave the resident state as the main workload left it
            device_step(W + K + i)
        torch.cuda.synchronize()

    # end to end through the host-buffer call: pinned ids -> device -> plan -> ranges on the host
    out_host = np.empty(1 << 16, dtype=capi.RANGE_DTYPE)
    e2e_ranges = 0
    for i in range(W):
        planner.step_host(h_slots[i % 2].numpy(), batches[i % 2].group_off,
                          batches[i % 2].budget_blocks, flags, out=out_host)
    barrier()
    t0 = time.perf_counter()
    for i in range(K):
        b = batches[(W + i) % 2]
        got, res = planner.step_host(h_slots[(W + i) % 2].numpy(), b.group_off, b.budget_blocks,
                                     flags, out=out_host)
        e2e_ranges = res.n_ranges
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / K
    plan = out_host[:e2e_ranges].copy()      # the last timed plan, compared across ranks below
    if variants:
        # the host-buffer call on int32 ids: half the bytes over the host link
        h32 = [torch.from_numpy(b.slots.astype(np.int32)).pin_memory() for b in batches]
        n32 = 20
        for i in range(2):
            planner.step_host(h32[i].numpy(), batches[i].group_off, batches[i].budget_blocks, flags,
                              out=out_host)
        t0 = time.perf_counter()
        for i in range(n32):
            b = batches[i % 2]
            planner.step_host(h32[i % 2].numpy(), b.group_off, b.budget_blocks, flags, out=out_host)
        torch.cuda.synchronize()
        variants["int32_ids_host_call"] = {"us_per_step": (time.perf_counter() - t0) / n32 * 1e6,
                                           "steps": n32, "h2d_bytes_per_step": 4 * batches[0].n_idx}
        del h32
        for i in range(2):      # back to the main pair's resident state
            planner.step_host(h_slots[(W + K + i) % 2].numpy(), batches[(W + K + i) % 2].group_off,
                              batches[(W + K + i) % 2].budget_blocks, flags, out=out_host)
    clocks = sampler.stop() if sampler else None

    ms_per_step, e2e_ms = ranks.max_over_ranks([total_ms / K, e2e_s * 1e3])
    launch_ms = ms_per_step           # one launch per step, nothing else on the stream
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
        achieved = bytes_step / (launch_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": ms_per_step * 1e3, "unit": UNIT, "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
            "config": workload_config(batches[0], {
                "parallelism": f"{world} independent per-GPU planners (one KV shard each), no collective on the data path",
                "l2": "178 MB of ids per step (> 126 MB L2); two batches alternate",
                "staging": "cp.async.bulk (TMA) -> shared" if args.tma else "ld.global 128-bit, two register sets",
                "launch": (f"CUDA graph of {per_replay} steps, replayed" if graph is not None
                           else "one launch per step on the stream") +
                          ("" if args.unchained else "; steps chained (programmatic dependent launch): "
                           "the scan of step i+1 runs over the tail of step i"),
                "evict": True}),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "traffic": PROFILED_TRAFFIC_BYTES.get((args.workload, bool(args.tma))),
                         "peak_source": peak_src, "algorithmic_bytes_per_launch": bytes_step,
                         "launch_ms": launch_ms, "kernel": "scan_plan_tma_kernel" if args.tma else "scan_plan_kernel"},
            "e2e": {"value": e2e_ms * 1e3, "unit": UNIT,
                    "h2d_bytes_per_step": 8 * batches[0].n_idx,
                    "d2h_bytes_per_step": 24 * e2e_ranges + 64},
            "gpu_launches": K,
            "clocks": clocks,
            "slot_scan_gbs_aggregate": world * achieved,
            "plans_per_s_aggregate": world / (ms_per_step * 1e-3),
            "ranges_per_step": n_ranges,
            "plans_agree_across_ranks": plans_agree,
        }
        if variants:
            line["variants"] = variants
            line["variants_launch"] = "one launch per step on the stream, 50 steps between two events"
        if cpu_lines:
            line.update(cpu_lines)
        emit(line)
    planner.close()
    ranks.stop()


# --------------------------------------------------------------------------
# event-driven path: device-resident feedback state, one plan per decode step
# --------------------------------------------------------------------------
def run_feedback(args):
    """--workload feedback: the incremental decode trace (65,536-slot pool, 40
    layers, Poisson arrivals, one token per live request per step) through
    rt_feedback_alloc / rt_feedback_attention / rt_feedback_plan, every index
    tensor already in HBM; beside it the Python restatement of
    SlotFeedback.consume -> publish -> target_blocks -> choose -> blocksv on one
    host core.  One GPU only."""
    import torch
    from retarget_b200 import capi, workloads
    from retarget_b200.feedback import DeviceFeedback
    from retarget_b200.planner import DevicePlanner, result_from_tensor

    K, W = args.steps, args.warmup
    layout = workloads.Layout(40, 2048, 65536)
    trace = workloads.decode_trace(0, steps=W + K, initial_requests=48)
    budget, max_blocks, active, refresh = 16, 16, 2.0, 10.0
    times = [100.0 + 0.03 * i for i in range(len(trace))]
    cpu = None
    if not args.no_cpu:
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
            out, _ = session.plan(times[i] + 0.001)
            if i >= W:
                t_cpu += time.perf_counter() - t0
                cpu_ranges += len(out)
        cpu = {"value": t_cpu / K * 1e6, "unit": UNIT, "cores": 1, "kind": "port",
               "sample": f"all {K} timed steps through the Python restatement of the reference's "
                         f"event-driven chain", "ranges": cpu_ranges}
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; retarget_b200 has no CPU path to fall back to")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    planner = DevicePlanner(layout, 0)
    fb = DeviceFeedback(planner, pid=0)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    d_steps = [(up(ev.alloc_slots) if len(ev.alloc_slots) else None,
                up(ev.free_head) if ev.free_head is not None and len(ev.alloc_slots) else None,
                up(ev.read_slots), up(ev.write_slots)) for ev in trace]
    d_out = torch.zeros((1 << 14) * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    h = stream.cuda_stream
    launches = 0

    def step(i):
        nonlocal launches
        a, head, r, w = d_steps[i]
        if a is not None:
            fb.alloc(a, times[i] - 0.002, head, h)
        fb.attention(r, w, times[i], h)
        fb.plan(times[i] + 0.001, budget=budget, max_blocks_per_update=max_blocks, active_seconds=active,
                refresh_seconds=refresh, flags=capi.RT_PLAN_EVICT, d_out=d_out, d_result=d_res, stream=h)

    sampler = ClockSampler(0)
    for i in range(W):
        step(i)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record(stream)
    gpu_ranges = 0
    for i in range(W, W + K):
        step(i)
    ev[1].record(stream)
    torch.cuda.synchronize()
    us = ev[0].elapsed_time(ev[1]) * 1e3 / K
    # same trace again, synchronising every step, to count the ranges and to
    # get the latency a caller sees (launch + run + read-back of the result)
    fb.clear(99.0, h)
    planner.set_resident([set()])
    t_sync = 0.0
    for i in range(W + K):
        t0 = time.perf_counter()
        step(i)
        stream.synchronize()
        n = result_from_tensor(d_res)["n_ranges"]
        if i >= W:
            t_sync += time.perf_counter() - t0
            gpu_ranges += n
    clocks = sampler.stop()
    ids = sum(len(e.alloc_slots) + len(e.read_slots) + len(e.write_slots) for e in trace[W:]) / K
    line = {"metric": "feedback_plan_us_per_decode_step", "value": us, "unit": UNIT, "n_gpus": 1, "steps": K,
            "warmup": W, "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "int64", "data": "synthetic",
            "config": {"workload": "incremental decode trace L40 S65536, event-driven feedback state",
                       "layers": 40, "pool_slots": 65536, "blocks_per_bitmap": layout.n_blocks,
                       "budget_blocks": budget, "event_ids_per_step": ids,
                       "live_requests_last_step": trace[-1].live},
            "e2e": {"value": t_sync / K * 1e6, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 64,
                    "note": "ids already on the device; launch + run + result read-back, one step at a time"},
            "ranges_total": gpu_ranges, "clocks": clocks}
    if cpu:
        line["cpu_baseline"] = cpu
        line["ranges_match_cpu"] = cpu["ranges"] == gpu_ranges
    emit(line)
    fb.close()
    planner.close()


# DRAM bytes per launch of the scan kernel from the ncu captures summarised under
# profiles/ (dram__bytes_read.sum + dram__bytes_write.sum, mean of 3 launches), keyed by
# (workload, tma); a configuration that was not captured reports null.
PROFILED_TRAFFIC_BYTES = {
    ("target", False): 181_694_000,   # 178.35 MB read + 3.35 MB written
    ("target", True): 182_228_000,    # 178.34 MB read + 3.89 MB written
}


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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="target",
                    choices=["target", "steady", "fragmented", "sparse", "full_refresh", "tp_shard", "feedback"])
    ap.add_argument("--tma", action="store_true", help="stage ids with bulk async copies (TMA)")
    ap.add_argument("--launch", default="graph", choices=["graph", "stream"],
                    help="how the timed launches are issued: CUDA graph replays or one by one")
    ap.add_argument("--unchained", action="store_true",
                    help="launch every step fully serialised after the one before it (no RT_PLAN_CHAINED)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-variants", action="store_true", help="skip the secondary measurements")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    quiet_stdout()
    if args.workload == "feedback":
        run_feedback(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
