#!/usr/bin/env python3
"""Regenerate the golden fixtures by running the UNMODIFIED reference modules.

Usage (needs the reference checkout; the fixtures it writes are committed so
the tests themselves never need it):

    python tests/golden/make_golden.py /path/to/reference

Writes ``tests/golden/reference_policy.json``: window/interval/run/mask/state
vectors from experiments/cache_window.py, slot_placement.py, slot_feedback.py
and kv_audit/kv_audit_probe.py, plus the command strings and accounting the two
controllers send to a recording stand-in for the UVM socket client.

Event timestamps are tie-free wherever a ranking is recorded: the reference
ranks with an unstable argsort, so ties would make the fixture depend on the
numpy build.
"""
import dataclasses
import importlib.util
import json
import os
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def load_reference(root):
    sys.path.insert(0, str(root))
    import experiments.cache_window as cw
    import experiments.slot_placement as sp
    import experiments.slot_feedback as sf
    import experiments.control as ctl
    spec = importlib.util.spec_from_file_location(
        "kv_audit_probe", Path(root) / "experiments/kv_audit/kv_audit_probe.py")
    probe = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(probe)
    return cw, sp, sf, ctl, probe


class RecordingUvm:
    """Stands in for UvmController: hands out a fixed allocation snapshot and
    records every command line."""

    def __init__(self, ctl, allocations, generation=7):
        self.ctl = ctl
        self.allocs = allocations
        self.generation = generation
        self.commands = []
        self.job = 0

    def _status(self):
        return self.ctl.UvmStatus(pid=1234, managed_bytes=sum(a["bytes"] for a in self.allocs),
                                  allocation_count=len(self.allocs),
                                  allocation_generation=self.generation, busy=False,
                                  job_id=self.job, completed_job=self.job, last_error=0,
                                  completed_cpu_bytes=0, completed_gpu_bytes=0,
                                  job_completed_bytes=0)

    def wait_idle(self, timeout=0):
        return self._status()

    def _allocation_snapshot(self):
        return self.generation, [dict(a) for a in self.allocs]

    def command(self, line):
        self.commands.append(line)
        self.job += 1
        return {"ok": True, "job_id": self.job}

    def _wait_job(self, job_id, timeout=0):
        return self._status()


def strip_times(d):
    """Drop wall-clock fields that differ between runs."""
    if d is None:
        return None
    d = dict(d)
    for k in ("audit_plan_committed_monotonic_s", "status"):
        d.pop(k, None)
    return d


def window_vectors(cw):
    specs = {
        "qwen": dict(allocation_bytes=448790528, allocation_count=80, bytes_per_token=2048),
        "llama": dict(allocation_bytes=297795584, allocation_count=120, bytes_per_token=2048,
                      width_tokens=21840, lookahead_tokens=10920, quantum_tokens=5460),
        "cfg1": dict(allocation_bytes=134217728, allocation_count=80, bytes_per_token=2048,
                     width_tokens=16384, lookahead_tokens=8192, quantum_tokens=1024),
        "cfg4": dict(allocation_bytes=67108864, allocation_count=96, bytes_per_token=256,
                     width_tokens=65536, lookahead_tokens=32768, quantum_tokens=8192),
        "odd": dict(allocation_bytes=1000000512, allocation_count=3, bytes_per_token=1536,
                    width_tokens=4096, lookahead_tokens=1024, quantum_tokens=8),
    }
    rng = np.random.default_rng(11)
    out = {}
    for name, kw in specs.items():
        s = cw.CacheWindowSpec(**kw)
        cap = kw["allocation_bytes"] // kw["bytes_per_token"]
        q = s.quantum_tokens
        probes = [0, 1, q - 1, q, q + 1, s.lookahead_tokens, s.lookahead_tokens + 1,
                  s.width_tokens, cap - 1, cap, cap + 1, 10 ** 9, 0.5, q - 0.25, 3 * q + 1e-9,
                  float(2 ** 53), 1e300]
        probes += [int(x) for x in rng.integers(0, 2 * cap, 40)]
        probes += [float(x) for x in rng.uniform(0, 1.5 * cap, 20)]
        out[name] = dict(spec=kw, cases=[[c, list(s.window(c))] for c in probes])
    bad = [
        (dict(allocation_bytes=448790528, allocation_count=80, bytes_per_token=2048,
              lookahead_tokens=32768), None),
        (dict(allocation_bytes=448790528, allocation_count=80, bytes_per_token=2048,
              quantum_tokens=3, width_tokens=3 * 1000, lookahead_tokens=3), None),
        (dict(allocation_bytes=448790528, allocation_count=80, bytes_per_token=2048,
              width_tokens=32768, lookahead_tokens=100, quantum_tokens=8192), None),
        (dict(allocation_bytes=4096, allocation_count=80, bytes_per_token=2048), None),
        (dict(allocation_bytes=0, allocation_count=80, bytes_per_token=2048), None),
        (dict(allocation_bytes=448790528, allocation_count=80, bytes_per_token=2048,
              min_update_seconds=-1.0), None),
        (dict(allocation_bytes=448790528, allocation_count=80, bytes_per_token=2048,
              idle_only=1), None),
        (dict(allocation_bytes=448790528, allocation_count=80, bytes_per_token=2048,
              update_mode="sometimes"), None),
        (dict(allocation_bytes=448790528, allocation_count=True, bytes_per_token=2048), None),
    ]
    rejected = []
    for kw, _ in bad:
        try:
            cw.CacheWindowSpec(**kw)
            rejected.append([kw, None])
        except ValueError as e:
            rejected.append([kw, str(e)])
    bad_counts = []
    s = cw.CacheWindowSpec(**specs["qwen"])
    for c in (-1, float("nan"), float("inf")):
        try:
            s.window(c)
            bad_counts.append([repr(c), None])
        except ValueError as e:
            bad_counts.append([repr(c), str(e)])
    pairs = [((0, 10), (5, 20)), ((5, 20), (0, 10)), ((0, 10), (20, 30)), ((0, 30), (10, 20)),
             ((0, 10), (0, 10)), ((4, 8), (0, 100)), ((0, 10), (10, 20)), ((10, 20), (0, 10)),
             ((7, 7), (0, 3)), ((0, 64), (0, 32)), ((0, 64), (32, 64))]
    pairs += [tuple(sorted(int(v) for v in rng.integers(0, 1000, 2)) for _ in range(2))
              for _ in range(60)]
    diffs = [[list(a), list(b), [list(p) for p in cw.interval_difference(tuple(a), tuple(b))]]
             for a, b in pairs]
    return dict(windows=out, rejected=rejected, bad_counts=bad_counts, interval_difference=diffs)


def run_vectors(probe, sp):
    rng = np.random.default_rng(5)
    cases = [[5, 6, 7, 7, 8, 3, 4, 10], [], [0], [-2, -1, 0, 1, 2], [9, 8, 7], [4, 4, 4]]
    for _ in range(20):
        n = int(rng.integers(1, 200))
        base = rng.integers(0, 5000, n)
        steps = rng.choice([1, 1, 1, 1, 0, 2, -1, 17], n)
        cases.append(np.cumsum(steps).astype(int).tolist() if rng.random() < .5
                     else (base // 16 * 16 + np.arange(n) % 16).astype(int).tolist())
    runs = [[c, probe.encode_runs(c)] for c in cases]
    masks = [[b, sp.encode_mask(b)] for b in
             ([], [0], [0, 5, 130], [1023], [3, 3, 3], list(range(64)),
              [int(x) for x in rng.integers(0, 1024, 40)])]
    return dict(encode_runs=runs, encode_mask=masks)


def feedback_vectors(sf, sp, probe):
    """Event streams through SlotFeedback and the ranking/selection functions."""
    out = []
    rng = np.random.default_rng(23)
    for case in range(6):
        T = [4, 16, 256, 1024, 8, 64][case]
        cap = [20, 500, 219135, 65535, 97, 4095][case]
        with tempfile.TemporaryDirectory() as tmp:
            fb = sf.SlotFeedback(tmp, pid=77, block_tokens=T, publish_seconds=1e9)
            events, snaps = [], []
            t = 100.0
            seq = 0
            n_events = 30
            for k in range(n_events):
                t += float(rng.uniform(0.01, 0.9))          # strictly increasing: no ties
                kind = rng.choice(["alloc", "attention", "attention", "alloc", "free"])
                if k == 0:
                    kind = "alloc"
                if k == 17 and case % 2:
                    kind = "allocator_clear"
                row = dict(event=str(kind), monotonic_s=t, sequence=seq)
                seq += 1

                def some_slots(count):
                    start = rng.integers(0, max(1, cap - 40), count)
                    vals = np.concatenate([np.arange(s, s + int(rng.integers(1, 40)))
                                           for s in start])
                    return np.clip(vals, 0, cap).astype(int).tolist()
                if kind == "alloc":
                    row["slot_runs"] = probe.encode_runs(some_slots(int(rng.integers(1, 4))))
                    row["allocator_size"] = cap
                    if rng.random() < .5:
                        row["free_head_runs"] = probe.encode_runs(some_slots(2))
                elif kind == "attention":
                    # one block per event keeps read/write stamps tie-free across blocks
                    b = int(rng.integers(0, (cap + T) // T))
                    lo = max(b * T, 0)
                    hi = min(lo + int(rng.integers(1, T + 1)), cap + 1)
                    row["read_runs"] = [[lo, hi]] if hi > lo else []
                    t += 0.001
                    row["write_runs"] = []
                elif kind == "allocator_clear":
                    row["allocator_size"] = cap
                else:
                    row["slot_runs"] = probe.encode_runs(some_slots(1))
                events.append(row)
                fb.consume(row)
                if fb.capacity:
                    fb.publish(t)
                    snap = json.loads((Path(tmp) / "77.json").read_text())
                    snap.pop("published_monotonic_s")
                    snaps.append(snap)
                else:
                    snaps.append(None)
            # ranking and selection on the last snapshot
            snap = snaps[-1]
            spec = sp.SlotPlacementSpec(block_tokens=T, max_blocks_per_update=3,
                                        active_seconds=2.0, refresh_seconds=1.5)
            picks = []
            for budget in (1, 2, 5, 1000):
                for now in (t, t + 1.0, t + 5.0, t + 40.0):
                    picks.append([budget, now, sp.target_blocks(snap, spec, budget, now)])
            out.append(dict(block_tokens=T, capacity=cap, events=events, snapshots=snaps,
                            versions=fb.versions.tolist(),
                            generations_sum=int(fb.generations.sum()),
                            target_blocks=picks))
    # blocks() known answers
    with tempfile.TemporaryDirectory() as tmp:
        fb = sf.SlotFeedback(tmp, pid=1, block_tokens=4)
        fb.reset(20)
        blocks = [[r, fb.blocks(r)] for r in
                  ([[0, 3], [9, 12], [2, 5]], [[0, 1]], [[-5, 2]], [[20, 21]], [[3, 3]], [[5, 4]],
                   [[1, 21]], [[8, 9], [4, 5], [0, 2]])]
    return dict(streams=out, blocks_T4_cap20=blocks)


def controller_vectors(cw, sp, sf, ctl):
    """Command strings + accounting from the two controllers."""
    out = {}
    kw = dict(allocation_bytes=134217728, allocation_count=8, bytes_per_token=2048,
              width_tokens=16384, lookahead_tokens=8192, quantum_tokens=1024,
              min_update_seconds=1.0, idle_only=True)
    allocs = ([dict(id=i + 1, bytes=134217728, device=0) for i in range(8)]
              + [dict(id=20, bytes=1 << 20, device=0), dict(id=21, bytes=12345 * 4096, device=0)])
    for mode in ("incremental", "full_cache", "initial_only"):
        spec = cw.CacheWindowSpec(update_mode=mode, **kw)
        c = cw.CacheWindowController(spec)
        uvm = RecordingUvm(ctl, allocs)
        log = []
        script = [  # (prompt, generation, running, queue, now, initial)
            (100, 0, 0, 0, 10.0, True), (5000, 100, 0, 0, 10.5, False),
            (9000, 200, 0, 0, 12.0, False), (9000, 200, 0, 0, 14.0, False),
            (20000, 900, 3, 0, 16.0, False), (20000, 900, 0, 0, 18.0, False),
            (10, 10, 0, 0, 20.0, False), (70000, 5000, 0, 0, 22.0, False),
            (90000, 5000, 0, 1, 24.0, False), (90000, 5000, 0, 0, 26.0, False)]
        for p, g, r, q, now, initial in script:
            m = {"sglang:prompt_tokens_total": float(p), "sglang:generation_tokens_total": float(g),
                 "sglang:num_running_reqs": float(r), "sglang:num_queue_reqs": float(q)}
            due = c.due(m, now)
            before = len(uvm.commands)
            res = c.update(uvm, m, now, initial=initial)
            log.append(dict(metrics=m, now=now, initial=initial, due=due,
                            commands=uvm.commands[before:], result=strip_times(res),
                            current=list(c.current) if c.current else None))
        # signature change forces a full plan
        if mode == "incremental":
            uvm.allocs = [dict(a, id=a["id"] + 100) for a in allocs]
            m = {"sglang:prompt_tokens_total": 95000.0, "sglang:generation_tokens_total": 5000.0,
                 "sglang:num_running_reqs": 0.0, "sglang:num_queue_reqs": 0.0}
            before = len(uvm.commands)
            res = c.update(uvm, m, 30.0)
            log.append(dict(metrics=m, now=30.0, initial=False, due=None,
                            commands=uvm.commands[before:], result=strip_times(res),
                            current=list(c.current), note="signature changed"))
            uvm.allocs = allocs[:-3]
            try:
                c.update(uvm, m, 40.0, initial=True)
                err = None
            except ctl.ControlError as e:
                err = str(e)
            log.append(dict(note="layout mismatch", error=err))
        out[mode] = dict(spec={**kw, "update_mode": mode}, allocations=allocs, generation=7,
                         log=log)
    return out


class FailingUvm(RecordingUvm):
    """RecordingUvm whose next command is rejected, or whose next job fails."""

    def __init__(self, ctl, allocations, generation=7):
        super().__init__(ctl, allocations, generation)
        self.reject_next = False
        self.fail_next_job = False

    def command(self, line):
        if self.reject_next:
            self.reject_next = False
            self.commands.append(line)
            return {"ok": False, "error": "busy"}
        return super().command(line)

    def _wait_job(self, job_id, timeout=0):
        if self.fail_next_job:
            self.fail_next_job = False
            raise self.ctl.ControlError(f"UVM job {job_id} for PID 1234 failed with CUDA error 700")
        return super()._wait_job(job_id, timeout)


def controller_failure_vectors(cw, sp, sf, ctl):
    """How the window controller reacts to metrics it cannot use, a command the
    socket rejects and a job that fails: the exception (type, text), the command
    lines sent, and the state afterwards."""
    kw = dict(allocation_bytes=134217728, allocation_count=8, bytes_per_token=2048,
              width_tokens=16384, lookahead_tokens=8192, quantum_tokens=1024,
              min_update_seconds=1.0, idle_only=True)
    allocs = [dict(id=i + 1, bytes=134217728, device=0) for i in range(8)] + [dict(id=20, bytes=1 << 20, device=0)]
    c = cw.CacheWindowController(cw.CacheWindowSpec(**kw))
    uvm = FailingUvm(ctl, allocs)
    full = {"sglang:prompt_tokens_total": 100.0, "sglang:generation_tokens_total": 0.0,
            "sglang:num_running_reqs": 0.0, "sglang:num_queue_reqs": 0.0}
    inf, nan = float("inf"), float("nan")
    script = [
        ("update", dict(full), 10.0, True, None),
        ("due", {k: v for k, v in full.items() if "prompt" not in k}, 12.0, False, None),
        ("update", {k: v for k, v in full.items() if "generation" not in k}, 12.0, False, None),
        ("update", dict(full, **{"sglang:prompt_tokens_total": -1.0}), 12.0, False, None),
        ("due", dict(full, **{"sglang:generation_tokens_total": inf}), 12.0, False, None),
        ("update", dict(full, **{"sglang:prompt_tokens_total": nan}), 12.0, False, None),
        # the gauges are looked up only when the window moved and the interval has passed
        ("due", {k: v for k, v in dict(full, **{"sglang:prompt_tokens_total": 9000.0}).items() if "running" not in k},
         12.0, False, None),
        ("update", {k: v for k, v in dict(full, **{"sglang:prompt_tokens_total": 9000.0}).items() if "queue" not in k},
         12.0, False, None),
        ("due", {k: v for k, v in full.items() if "running" not in k}, 12.0, False, None),      # window unchanged
        ("update", dict(full, **{"sglang:prompt_tokens_total": 9000.0}), 12.0, False, "reject"),
        ("update", dict(full, **{"sglang:prompt_tokens_total": 9000.0}), 12.5, False, "fail_job"),
        ("update", dict(full, **{"sglang:prompt_tokens_total": 9000.0}), 13.0, False, None),    # state was dropped: full plan
        ("update", dict(full, **{"sglang:prompt_tokens_total": 30000.0}), 15.0, False, None),
    ]
    log = []
    for op, m, now, initial, trouble in script:
        uvm.reject_next, uvm.fail_next_job = trouble == "reject", trouble == "fail_job"
        before = len(uvm.commands)
        entry = dict(op=op, metrics={k: (repr(v) if v != v or v in (inf, -inf) else v) for k, v in m.items()},
                     now=now, initial=initial, trouble=trouble)
        try:
            got = c.due(m, now) if op == "due" else strip_times(c.update(uvm, m, now, initial=initial))
            entry["result"] = got
        except Exception as e:                                   # noqa: BLE001 -- the type is the datum
            entry["error"] = [type(e).__name__, str(e) if not isinstance(e, KeyError) else e.args[0]]
        entry["commands"] = uvm.commands[before:]
        entry["current"] = list(c.current) if c.current else None
        entry["signature_known"] = c.signature is not None
        entry["highwater"] = c.completed_highwater
        log.append(entry)
    return dict(spec=kw, allocations=allocs, generation=7, log=log)


def placement_controller_vectors(cw, sp, sf, ctl):
    """SlotPlacementController.choose/update against hand-built snapshots."""
    kw = dict(allocation_bytes=16 * 2097152, allocation_count=4, bytes_per_token=2048,
              width_tokens=4096, lookahead_tokens=1024, quantum_tokens=1024)
    allocs = [dict(id=i + 1, bytes=16 * 2097152, device=0) for i in range(4)] + \
             [dict(id=9, bytes=4096, device=0)]
    sspec = dict(block_tokens=1024, lookahead_tokens=4096, min_update_seconds=.25,
                 max_blocks_per_update=2, active_seconds=2.0, refresh_seconds=10.0,
                 max_feedback_lag_seconds=1.0)
    log = []
    with tempfile.TemporaryDirectory() as tmp:
        os.environ["RETARGET_SLOT_FEEDBACK_DIR"] = tmp
        c = sp.SlotPlacementController(cw.CacheWindowSpec(**kw), sp.SlotPlacementSpec(**sspec), 4242)
        c.signature = tuple((a["id"], a["bytes"], a["device"]) for a in allocs[:4])
        c.epoch = 1
        uvm = RecordingUvm(ctl, allocs)
        path = Path(tmp) / "4242.json"

        def snap(now, reads, writes, free, versions, epoch=1, lag=0.0, seq=0):
            d = dict(version=1, pid=4242, epoch=epoch, sequence=seq,
                     observed_monotonic_s=now - lag, published_monotonic_s=now,
                     capacity_tokens=16383, block_tokens=1024, block_versions=versions,
                     recent_reads=reads, recent_writes=writes, free_head_blocks=free)
            path.write_text(json.dumps(d))
            return d
        v = [0] * 16
        steps = [
            (50.0, [[3, 49.9], [7, 49.5], [1, 40.0]], [[9, 49.8]], [12, 3], v, 1, 0.0),
            (50.1, [[3, 49.9], [7, 49.5], [1, 40.0]], [[9, 49.8]], [12, 3], v, 1, 0.0),
            (50.5, [[3, 49.9], [7, 49.5], [1, 40.0]], [[9, 49.8]], [12, 3], v, 1, 0.0),
            (51.0, [[3, 49.9], [7, 49.5], [1, 40.0]], [[9, 49.8]], [12, 3], v, 1, 0.0),
            (52.0, [[5, 51.9], [3, 49.9]], [[9, 51.5]], [], [0, 0, 0, 2] + [0] * 12, 1, 0.0),
            (53.0, [[5, 52.9]], [], [], v, 1, 5.0),
            (54.0, [[2, 53.9], [5, 52.9]], [], [14], v, 2, 0.0),
            (70.0, [[2, 69.9]], [], [], v, 2, 0.0),
        ]
        # The controller stamps commits with time.monotonic(); pin that clock to the
        # scripted time so the refresh rule is exercised reproducibly.
        clock = {"now": 0.0}
        real_time = sp.time

        class ScriptedTime:
            @staticmethod
            def monotonic():
                return clock["now"]
        sp.time = ScriptedTime
        for now, reads, writes, free, versions, epoch, lag in steps:
            clock["now"] = now
            s = snap(now, reads, writes, free, versions, epoch, lag)
            m = {"sglang:prompt_tokens_total": 0.0, "sglang:generation_tokens_total": 0.0}
            due = c.due(m, now)
            before = len(uvm.commands)
            res = c.update(uvm, m, now)
            if res is not None:
                res = {k: res[k] for k in ("desired_blocks", "gpu_blocks", "committed_blocks",
                                           "requested_gpu_bytes", "requested_cpu_bytes",
                                           "feedback_epoch", "allocation_generation")}
            log.append(dict(snapshot=s, now=now, due=due, commands=uvm.commands[before:],
                            result=res, committed_versions={str(k): val[0]
                                                            for k, val in c.committed.items()}))
        sp.time = real_time
    return dict(cache_spec=kw, slot_spec=sspec, allocations=allocs, generation=7, pid=4242, log=log)


def placement_failure_vectors(cw, sp, sf, ctl):
    """SlotPlacementController when things go wrong: no snapshot file, a snapshot
    of another process or geometry, a stale one, a rejected command, a failed
    job, another set of cache allocations, too few of them."""
    kw = dict(allocation_bytes=16 * 2097152, allocation_count=4, bytes_per_token=2048,
              width_tokens=4096, lookahead_tokens=1024, quantum_tokens=1024)
    allocs = [dict(id=i + 1, bytes=16 * 2097152, device=0) for i in range(4)] + [dict(id=9, bytes=4096, device=0)]
    sspec = dict(block_tokens=1024, lookahead_tokens=4096, min_update_seconds=.25,
                 max_blocks_per_update=2, active_seconds=2.0, refresh_seconds=10.0,
                 max_feedback_lag_seconds=1.0)
    log = []
    clock = {"now": 0.0}

    class ScriptedTime:
        @staticmethod
        def monotonic():
            return clock["now"]
    real_time = sp.time
    sp.time = ScriptedTime
    try:
        with tempfile.TemporaryDirectory() as tmp:
            os.environ["RETARGET_SLOT_FEEDBACK_DIR"] = tmp
            c = sp.SlotPlacementController(cw.CacheWindowSpec(**kw), sp.SlotPlacementSpec(**sspec), 4242)
            c.signature = tuple((a["id"], a["bytes"], a["device"]) for a in allocs[:4])
            c.epoch = 1
            uvm = FailingUvm(ctl, allocs)
            path = Path(tmp) / "4242.json"

            def doc(now, reads, free, **over):
                d = dict(version=1, pid=4242, epoch=1, sequence=0, observed_monotonic_s=now,
                         published_monotonic_s=now, capacity_tokens=16383, block_tokens=1024,
                         block_versions=[0] * 16, recent_reads=reads, recent_writes=[], free_head_blocks=free)
                d.update(over)
                return d
            steps = [
                (50.0, None, None, None),                                                   # no file yet
                (50.5, doc(50.5, [[3, 50.4]], [], pid=7), None, None),                       # another process
                (51.0, doc(51.0, [[3, 50.9]], [], block_tokens=256), None, None),            # another geometry
                (51.5, doc(51.5, [[3, 51.4]], [], observed_monotonic_s=49.0), None, None),   # published late
                (52.0, doc(52.0, [[3, 51.9], [5, 51.8]], [7]), "reject", None),
                (52.5, doc(52.5, [[3, 52.4], [5, 52.3]], [7]), "fail_job", None),
                (53.0, doc(53.0, [[3, 52.9], [5, 52.8]], [7]), None, None),                  # record was dropped: again
                (53.5, doc(53.5, [[3, 53.4], [5, 53.3]], [7]), None, None),
                (54.0, doc(54.0, [[3, 53.9], [5, 53.8], [6, 53.7]], [7]), None, "renumber"),  # other allocation ids
                (54.5, doc(54.5, [[3, 54.4], [5, 54.3], [6, 54.2], [8, 54.1]], [7]), None, "drop_one"),
            ]
            for now, snapshot, trouble, registry in steps:
                clock["now"] = now
                if snapshot is None:
                    if path.exists():
                        path.unlink()
                else:
                    path.write_text(json.dumps(snapshot))
                if registry == "renumber":
                    uvm.allocs = [dict(a, id=a["id"] + 40) for a in allocs]
                elif registry == "drop_one":
                    uvm.allocs = uvm.allocs[1:]
                uvm.reject_next, uvm.fail_next_job = trouble == "reject", trouble == "fail_job"
                m = {"sglang:prompt_tokens_total": 0.0, "sglang:generation_tokens_total": 0.0}
                entry = dict(now=now, snapshot=snapshot, trouble=trouble, registry=registry)
                before = len(uvm.commands)
                for op in ("due", "update"):
                    try:
                        got = c.due(m, now) if op == "due" else c.update(uvm, m, now)
                        if op == "update" and got is not None:
                            got = {k: got[k] for k in ("desired_blocks", "gpu_blocks", "committed_blocks",
                                                       "requested_gpu_bytes")}
                        entry[op] = got
                    except Exception as e:                       # noqa: BLE001 -- the type is the datum
                        entry[op + "_error"] = [type(e).__name__, str(e)]
                entry["commands"] = uvm.commands[before:]
                entry["committed"] = sorted(c.committed)
                entry["last_attempt"] = c.last_attempt
                log.append(entry)
    finally:
        sp.time = real_time
    return dict(cache_spec=kw, slot_spec=sspec, allocations=allocs, generation=7, pid=4242, log=log)


def placement_chain_vectors(cw, sp, sf, ctl, probe):
    """The whole event-driven chain of the reference, unmodified: event rows ->
    SlotFeedback.consume/publish (snapshot file) -> SlotPlacementController.update,
    over a scripted 45 s during which committed blocks drop out of the desired set
    while nothing is selected (their stamps age past the 30 s horizon; the sampled
    free-list head moves away) and later come back with their versions unchanged.
    The controller must not send them again: it returns before it touches
    ``committed`` when nothing was selected.  Stamps are tie-free."""
    kw = dict(allocation_bytes=16 * 2097152, allocation_count=4, bytes_per_token=2048,
              width_tokens=4096, lookahead_tokens=1024, quantum_tokens=1024)
    allocs = [dict(id=i + 1, bytes=16 * 2097152, device=0) for i in range(4)]
    sspec = dict(block_tokens=1024, lookahead_tokens=4096, min_update_seconds=.25,
                 max_blocks_per_update=2, active_seconds=2.0, refresh_seconds=1000.0,
                 max_feedback_lag_seconds=1.0)
    cap = 16383
    # (time, kind, fields); "update" rows call the controller at that time
    script = [
        (100.00, "alloc", dict(slots=list(range(1, 200)), free_head=list(range(5000, 5010)))),
        (100.05, "alloc", dict(slots=list(range(1100, 1300)))),
        (100.10, "attention", dict(read=list(range(10, 20)), write=[])),
        (100.20, "attention", dict(read=list(range(1100, 1200)), write=[])),
        (100.30, "update", {}),          # desired [1, 0, 4]: the first two are sent
        (100.60, "update", {}),          # block 4 follows
        (100.90, "update", {}),          # nothing to do
        # the sampled free head moves into block 0: block 4 is no longer desired, nothing is selected
        (101.00, "alloc", dict(slots=[], free_head=list(range(100, 110)))),
        (101.30, "update", {}),
        # ... and comes back: block 4 is desired again, still committed, version unchanged
        (101.50, "alloc", dict(slots=[], free_head=list(range(5000, 5010)))),
        (101.80, "update", {}),
        # 30 s later every stamp has aged out: only the free head is desired
        (131.00, "free", dict(slots=[7000])),
        (131.30, "update", {}),
        # block 0 is read again: desired, still committed, version unchanged
        (132.00, "attention", dict(read=list(range(30, 40)), write=[])),
        (132.30, "update", {}),
        # a re-allocation bumps block 1's version: this one is sent again
        (133.00, "alloc", dict(slots=list(range(1100, 1110)))),
        (133.30, "update", {}),
        # a new block becomes active: sent, and what is no longer desired is dropped
        (140.00, "attention", dict(read=list(range(9300, 9310)), write=list(range(12300, 12301)))),
        (140.30, "update", {}),
        (140.60, "update", {}),
        (145.00, "attention", dict(read=list(range(5005, 5006)), write=[])),
        (145.30, "update", {}),
    ]
    log = []
    clock = {"now": 0.0}

    class ScriptedTime:
        @staticmethod
        def monotonic():
            return clock["now"]
    real_sp, real_sf = sp.time, sf.time
    sp.time = sf.time = ScriptedTime
    try:
        with tempfile.TemporaryDirectory() as tmp:
            os.environ["RETARGET_SLOT_FEEDBACK_DIR"] = tmp
            fb = sf.SlotFeedback(tmp, pid=4242, block_tokens=1024, publish_seconds=0.0)
            c = sp.SlotPlacementController(cw.CacheWindowSpec(**kw), sp.SlotPlacementSpec(**sspec), 4242)
            c.signature = tuple((a["id"], a["bytes"], a["device"]) for a in allocs)
            c.epoch = 1
            uvm = RecordingUvm(ctl, allocs)
            seq = 0
            for t, kind, f in script:
                clock["now"] = t
                if kind == "update":
                    m = {"sglang:prompt_tokens_total": 0.0, "sglang:generation_tokens_total": 0.0}
                    before = len(uvm.commands)
                    res = c.update(uvm, m, t)
                    if res is not None:
                        res = {k: res[k] for k in ("desired_blocks", "gpu_blocks", "committed_blocks",
                                                   "requested_gpu_bytes")}
                    log.append(dict(t=t, kind=kind, commands=uvm.commands[before:], result=res,
                                    committed=sorted(c.committed),
                                    committed_versions={str(k): v[0] for k, v in c.committed.items()}))
                    continue
                row = dict(event=kind, monotonic_s=t, sequence=seq)
                seq += 1
                if kind == "alloc":
                    row["slot_runs"] = probe.encode_runs(f["slots"])
                    row["allocator_size"] = cap
                    if "free_head" in f:
                        row["free_head_runs"] = probe.encode_runs(f["free_head"])
                elif kind == "attention":
                    row["read_runs"] = probe.encode_runs(f["read"])
                    row["write_runs"] = probe.encode_runs(f["write"])
                else:
                    row["slot_runs"] = probe.encode_runs(f["slots"])
                fb.consume(row)
                log.append(dict(t=t, kind=kind, fields=f))
    finally:
        sp.time, sf.time = real_sp, real_sf
    return dict(cache_spec=kw, slot_spec=sspec, capacity=cap, allocations=allocs, generation=7, pid=4242,
                log=log)


TARGET_SCRIPT = [
    # (operation, arguments) against the scripted transport below
    ("set_target", dict(gpu_bytes=0)),
    ("set_target", dict(gpu_bytes=50 * (1 << 20) + 1234)),
    ("retarget", dict(previous_gpu_bytes=50 * (1 << 20) + 1234, gpu_bytes=12 * (1 << 20))),
    ("retarget", dict(previous_gpu_bytes=1, gpu_bytes=13 * (1 << 20) + 5)),          # stale previous
    ("bump_generation", dict()),
    ("retarget", dict(previous_gpu_bytes=13 * (1 << 20) + 5, gpu_bytes=70 * (1 << 20))),  # registry changed
    ("set_target", dict(gpu_bytes=1 << 40)),                                           # clamped
    ("set_target", dict(gpu_bytes=3 * (1 << 20), wait=False)),
    ("wait_idle", dict()),
    ("retarget", dict(previous_gpu_bytes=3 * (1 << 20), gpu_bytes=9 * (1 << 20) + 777, wait=False)),
    ("wait_idle", dict()),
    ("retarget", dict(previous_gpu_bytes=9 * (1 << 20) + 777, gpu_bytes=2 * (1 << 20))),
    ("reject_next", dict(error="busy")),
    ("retarget", dict(previous_gpu_bytes=2 * (1 << 20), gpu_bytes=5 * (1 << 20))),
    ("fail_next_job", dict(code=700)),
    ("retarget", dict(previous_gpu_bytes=2 * (1 << 20), gpu_bytes=6 * (1 << 20))),
    ("retarget", dict(previous_gpu_bytes=6 * (1 << 20), gpu_bytes=7 * (1 << 20))),     # state was dropped
    ("fail_next_job", dict(code=2)),
    ("set_target", dict(gpu_bytes=8 * (1 << 20), wait=False)),
    ("wait_idle", dict()),
    ("retarget", dict(previous_gpu_bytes=8 * (1 << 20), gpu_bytes=1 << 20)),
    ("set_target", dict(gpu_bytes=-1)),
]
TARGET_ALLOCATIONS = [dict(id=3, bytes=10 * (1 << 20) + 100, device=0), dict(id=4, bytes=64 * (1 << 20), device=0),
                      dict(id=9, bytes=4 * (1 << 20) + 3 * 4096, device=1)]


class ScriptedServer:
    """Answers status / list / plan lines like the preload library's socket would,
    completing every accepted job at once."""

    def __init__(self, pid, allocations):
        self.pid, self.allocs, self.generation = pid, [dict(a) for a in allocations], 5
        self.job, self.last_error, self.reject, self.fail_code = 0, 0, None, 0
        self.lines = []

    def __call__(self, line):
        self.lines.append(line)
        if line == "status":
            return dict(ok=True, pid=self.pid, managed_bytes=sum(a["bytes"] for a in self.allocs),
                        allocation_count=len(self.allocs), allocation_generation=self.generation, busy=False,
                        job_id=self.job, completed_job=self.job, last_error=self.last_error,
                        completed_cpu_bytes=0, completed_gpu_bytes=0, job_completed_bytes=0)
        if line == "list":
            return dict(ok=True, allocation_generation=self.generation, allocations=[dict(a) for a in self.allocs])
        if self.reject:
            error, self.reject = self.reject, None
            return dict(ok=False, error=error)
        self.job += 1
        self.last_error, self.fail_code = self.fail_code, 0
        return dict(ok=True, job_id=self.job)


def run_target_script(make_controller, ControlError, page):
    """Shared by the generator (reference controller) and the replay test."""
    server = ScriptedServer(os.getpid(), TARGET_ALLOCATIONS)
    c = make_controller(server)
    log = []
    for op, kw in TARGET_SCRIPT:
        before = len(server.lines)
        entry = dict(op=op, args=kw)
        if op == "bump_generation":
            server.generation += 1
            server.allocs.append(dict(id=12, bytes=8 * page, device=0))
        elif op == "reject_next":
            server.reject = kw["error"]
        elif op == "fail_next_job":
            server.fail_code = kw["code"]
        else:
            try:
                res = getattr(c, op)(**kw)
                if dataclasses.is_dataclass(res):
                    kind = type(res).__name__
                    res = {k: v for k, v in dataclasses.asdict(res).items() if k != "status"}
                    res["type"] = kind
                entry["result"] = res
            except (ControlError, ValueError) as e:
                entry["error"] = [type(e).__name__, str(e)]
        entry["lines"] = server.lines[before:]
        entry["submitted_target"] = getattr(c, "_submitted_target", None)
        entry["pending_job"] = getattr(c, "_pending_job", None)
        log.append(entry)
    return log


def target_vectors(ctl):
    """aligned_uvm_target, and UvmController.set_target / retarget / wait_idle
    driven through a scripted transport (control.py:379-400,488-654)."""
    rng = np.random.default_rng(4)
    aligned = []
    for _ in range(200):
        page = int(rng.choice([4096, 65536]))
        sizes = [int(rng.integers(0, 40) * page + rng.choice([0, 0, 100, page // 2])) for _ in range(rng.integers(0, 6))]
        total = sum(sizes)
        desired = int(rng.integers(0, total + 3 * page + 1))
        aligned.append([sizes, desired, page, ctl.aligned_uvm_target(sizes, desired, page)])
    page = os.sysconf("SC_PAGE_SIZE")

    def make(server):
        c = ctl.UvmController(os.getpid())
        c.command = server
        return c
    return dict(aligned=aligned, page=page, pid=os.getpid(),
                script=run_target_script(make, ctl.ControlError, page))



def main():
    root = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["RETARGET_REFERENCE"])
    cw, sp, sf, ctl, probe = load_reference(root)
    doc = dict(
        generated_by="tests/golden/make_golden.py (unmodified reference modules)",
        numpy=np.__version__,
        window=window_vectors(cw),
        runs=run_vectors(probe, sp),
        feedback=feedback_vectors(sf, sp, probe),
        window_controller=controller_vectors(cw, sp, sf, ctl),
        controller_failures=controller_failure_vectors(cw, sp, sf, ctl),
        placement_controller=placement_controller_vectors(cw, sp, sf, ctl),
        placement_failures=placement_failure_vectors(cw, sp, sf, ctl),
        placement_chain=placement_chain_vectors(cw, sp, sf, ctl, probe),
        targets=target_vectors(ctl),
    )
    path = HERE / "reference_policy.json"
    path.write_text(json.dumps(doc, separators=(",", ":"), allow_nan=True))
    print("wrote", path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
