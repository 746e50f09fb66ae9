"""The scheduler-facing controllers replayed against logs recorded from the
reference controllers (same metrics, same clock, same registry): every command
line, every gate decision and every accounting field must match."""
import json

import pytest

from retarget_b200 import cache_window as cw
from retarget_b200 import slot_placement as sp
from retarget_b200.control import ControlError, UvmStatus


class RecordingUvm:
    def __init__(self, allocations, generation):
        self.allocs, self.generation, self.commands, self.job = allocations, generation, [], 0

    def _status(self):
        return UvmStatus(1234, sum(a["bytes"] for a in self.allocs), len(self.allocs), self.generation,
                         False, self.job, self.job, 0, 0, 0, 0)

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


def _strip(result):
    if result is None:
        return None
    result = dict(result)
    result.pop("audit_plan_committed_monotonic_s", None)
    result.pop("status", None)
    return result


def test_spec_validation_matches_reference(golden):
    for kw, message in golden["window"]["rejected"]:
        with pytest.raises(ValueError) as e:
            cw.CacheWindowSpec(**kw)
        assert str(e.value) == message
    spec = cw.CacheWindowSpec(448790528, 80, 2048)
    for text, message in golden["window"]["bad_counts"]:
        with pytest.raises(ValueError) as e:
            spec.window(float(text))
        assert str(e.value) == message
    for name, block in golden["window"]["windows"].items():
        s = cw.CacheWindowSpec(**block["spec"])
        for c, want in block["cases"]:
            assert list(s.window(c)) == want
    for a, b, want in golden["window"]["interval_difference"]:
        assert [list(p) for p in cw.interval_difference(tuple(a), tuple(b))] == want
    for blocks, want in golden["runs"]["encode_mask"]:
        assert sp.encode_mask(blocks) == want
    with pytest.raises(ValueError, match="block_tokens"):
        sp.SlotPlacementSpec(block_tokens=0)
    with pytest.raises(ValueError, match="refresh_seconds"):
        sp.SlotPlacementSpec(refresh_seconds=float("inf"))


def test_window_controller_replay(golden):
    for mode, block in golden["window_controller"].items():
        ctl = cw.CacheWindowController(cw.CacheWindowSpec(**block["spec"]))
        uvm = RecordingUvm(block["allocations"], block["generation"])
        for step in block["log"]:
            note = step.get("note")
            if note == "signature changed":
                uvm.allocs = [dict(a, id=a["id"] + 100) for a in block["allocations"]]
            if note == "layout mismatch":
                uvm.allocs = block["allocations"][:-3]
                with pytest.raises(ControlError) as e:
                    ctl.update(uvm, metrics, 40.0, initial=True)
                assert str(e.value) == step["error"]
                continue
            metrics, now = step["metrics"], step["now"]
            if step["due"] is not None:
                assert ctl.due(metrics, now) == step["due"], (mode, now)
            before = len(uvm.commands)
            got = ctl.update(uvm, metrics, now, initial=step["initial"])
            assert uvm.commands[before:] == step["commands"], (mode, now)
            assert _strip(got) == step["result"], (mode, now)
            assert (list(ctl.current) if ctl.current else None) == step["current"]


class FailingUvm(RecordingUvm):
    def __init__(self, allocations, generation):
        super().__init__(allocations, generation)
        self.reject_next = self.fail_next_job = False

    def command(self, line):
        if self.reject_next:
            self.reject_next = False
            self.commands.append(line)
            return {"ok": False, "error": "busy"}
        return super().command(line)

    def _wait_job(self, job_id, timeout=0):
        if self.fail_next_job:
            self.fail_next_job = False
            raise ControlError(f"UVM job {job_id} for PID 1234 failed with CUDA error 700")
        return super()._wait_job(job_id, timeout)


def test_window_controller_failures_replay(golden):
    """Metrics the policy cannot use (a counter missing, negative, infinite, NaN; a
    gauge missing when it is needed), a command the socket rejects and a job that
    fails: same exception type and text, same lines on the wire and same state
    afterwards as the reference controller."""
    block = golden["controller_failures"]
    ctl = cw.CacheWindowController(cw.CacheWindowSpec(**block["spec"]))
    uvm = FailingUvm(block["allocations"], block["generation"])
    kinds = {"ControlError": ControlError, "KeyError": KeyError, "ValueError": ValueError}
    for step in block["log"]:
        metrics = {k: (float(v.strip("'")) if isinstance(v, str) else v) for k, v in step["metrics"].items()}
        uvm.reject_next, uvm.fail_next_job = step["trouble"] == "reject", step["trouble"] == "fail_job"
        before = len(uvm.commands)

        def call():
            if step["op"] == "due":
                return ctl.due(metrics, step["now"])
            return _strip(ctl.update(uvm, metrics, step["now"], initial=step["initial"]))
        if "error" in step:
            kind, text = step["error"]
            with pytest.raises(kinds[kind]) as e:
                call()
            assert (e.value.args[0] if kind == "KeyError" else str(e.value)) == text, step
        else:
            assert call() == step["result"], step
        assert uvm.commands[before:] == step["commands"]
        assert (list(ctl.current) if ctl.current else None) == step["current"]
        assert (ctl.signature is not None) == step["signature_known"]
        assert ctl.completed_highwater == step["highwater"]


def test_placement_controller_replay(golden, tmp_path, monkeypatch):
    block = golden["placement_controller"]
    monkeypatch.setenv("RETARGET_SLOT_FEEDBACK_DIR", str(tmp_path))
    clock = {"now": 0.0}

    class Scripted:
        @staticmethod
        def monotonic():
            return clock["now"]
    monkeypatch.setattr(sp, "time", Scripted)
    ctl = sp.SlotPlacementController(cw.CacheWindowSpec(**block["cache_spec"]),
                                     sp.SlotPlacementSpec(**block["slot_spec"]), block["pid"])
    n_cache = block["cache_spec"]["allocation_count"]
    ctl.signature = tuple((a["id"], a["bytes"], a["device"]) for a in block["allocations"][:n_cache])
    ctl.epoch = 1
    uvm = RecordingUvm(block["allocations"], block["generation"])
    keys = ("desired_blocks", "gpu_blocks", "committed_blocks", "requested_gpu_bytes",
            "requested_cpu_bytes", "feedback_epoch", "allocation_generation")
    for step in block["log"]:
        clock["now"] = step["now"]
        (tmp_path / f"{block['pid']}.json").write_text(json.dumps(step["snapshot"]))
        metrics = {"sglang:prompt_tokens_total": 0.0, "sglang:generation_tokens_total": 0.0}
        assert ctl.due(metrics, step["now"]) == step["due"]
        before = len(uvm.commands)
        got = ctl.update(uvm, metrics, step["now"])
        assert uvm.commands[before:] == step["commands"]
        assert (None if got is None else {k: got[k] for k in keys}) == step["result"]
        assert {str(k): v[0] for k, v in ctl.committed.items()} == step["committed_versions"]
    # the same controller fed by a callable instead of the file drop
    ctl2 = sp.SlotPlacementController(cw.CacheWindowSpec(**block["cache_spec"]),
                                      sp.SlotPlacementSpec(**block["slot_spec"]), block["pid"],
                                      snapshot_source=lambda now: block["log"][0]["snapshot"])
    assert ctl2.choose(ctl2.snapshot(50.0), 50.0) == ([3, 7, 9, 12], [3, 7])


def test_placement_controller_failures_replay(golden, tmp_path, monkeypatch):
    """No snapshot file, a snapshot of another process or geometry, a stale one, a
    rejected command, a failed job, renumbered allocations, a missing allocation:
    same answers, exceptions, lines and record as the reference controller."""
    block = golden["placement_failures"]
    monkeypatch.setenv("RETARGET_SLOT_FEEDBACK_DIR", str(tmp_path))
    clock = {"now": 0.0}

    class Scripted:
        @staticmethod
        def monotonic():
            return clock["now"]
    monkeypatch.setattr(sp, "time", Scripted)
    ctl = sp.SlotPlacementController(cw.CacheWindowSpec(**block["cache_spec"]),
                                     sp.SlotPlacementSpec(**block["slot_spec"]), block["pid"])
    ctl.signature = tuple((a["id"], a["bytes"], a["device"]) for a in block["allocations"][:4])
    ctl.epoch = 1
    uvm = FailingUvm(block["allocations"], block["generation"])
    path = tmp_path / f"{block['pid']}.json"
    keys = ("desired_blocks", "gpu_blocks", "committed_blocks", "requested_gpu_bytes")
    for step in block["log"]:
        clock["now"] = now = step["now"]
        if step["snapshot"] is None:
            path.unlink(missing_ok=True)
        else:
            path.write_text(json.dumps(step["snapshot"]))
        if step["registry"] == "renumber":
            uvm.allocs = [dict(a, id=a["id"] + 40) for a in block["allocations"]]
        elif step["registry"] == "drop_one":
            uvm.allocs = uvm.allocs[1:]
        uvm.reject_next, uvm.fail_next_job = step["trouble"] == "reject", step["trouble"] == "fail_job"
        metrics = {"sglang:prompt_tokens_total": 0.0, "sglang:generation_tokens_total": 0.0}
        before = len(uvm.commands)
        for op in ("due", "update"):
            def call():
                if op == "due":
                    return ctl.due(metrics, now)
                got = ctl.update(uvm, metrics, now)
                return None if got is None else {k: got[k] for k in keys}
            if op + "_error" in step:
                with pytest.raises(ControlError) as e:
                    call()
                assert [type(e.value).__name__, str(e.value)] == step[op + "_error"], (now, op)
            else:
                assert call() == step[op], (now, op)
        assert uvm.commands[before:] == step["commands"], now
        assert sorted(ctl.committed) == step["committed"], now
        assert ctl.last_attempt == step["last_attempt"], now


def test_budget_rules():
    with pytest.raises(ValueError, match="KV budget must be divisible by block_tokens"):
        sp.SlotPlacementController(cw.CacheWindowSpec(16 * 2097152, 4, 2048, 4096, 1024, 1024),
                                   sp.SlotPlacementSpec(block_tokens=3000), 1, snapshot_source=lambda n: None)
    with pytest.raises(ValueError, match="slot blocks must be page aligned"):
        sp.SlotPlacementController(cw.CacheWindowSpec(16 * 2097152, 4, 4, 4096, 1024, 1024),
                                   sp.SlotPlacementSpec(block_tokens=512), 1, snapshot_source=lambda n: None)


def _golden_tools():
    import importlib.util
    from pathlib import Path
    path = Path(__file__).resolve().parent / "golden" / "make_golden.py"
    spec = importlib.util.spec_from_file_location("make_golden", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_aligned_target_matches_reference(golden):
    from retarget_b200.control import aligned_uvm_target
    for sizes, desired, page, want in golden["targets"]["aligned"]:
        assert aligned_uvm_target(sizes, desired, page) == want
    with pytest.raises(ValueError):
        aligned_uvm_target([4096], -1, 4096)
    with pytest.raises(ValueError):
        aligned_uvm_target([4096, -2], 0, 4096)
    with pytest.raises(ValueError):
        aligned_uvm_target([4096], 0, 0)


def test_prefix_plans_replay(golden):
    """set_target / retarget / wait_idle against the scripted transport the
    reference client was recorded with: same lines on the wire, same results,
    same errors, same remembered placement after every call."""
    import os
    from retarget_b200.control import UvmController
    tools = _golden_tools()
    block = golden["targets"]
    assert block["page"] == os.sysconf("SC_PAGE_SIZE")

    def make(server):
        c = UvmController(os.getpid())
        c.command = server
        return c

    got = tools.run_target_script(make, ControlError, block["page"])
    theirs, ours = str(block["pid"]), str(os.getpid())
    assert len(got) == len(block["script"])
    for mine, want in zip(got, block["script"]):
        want = json.loads(json.dumps(want))
        if "error" in want:                       # the messages name the controlled PID
            want["error"][1] = want["error"][1].replace(f"PID {theirs}", f"PID {ours}")
        if isinstance(want.get("result"), dict) and "pid" in want["result"]:
            want["result"]["pid"] = int(ours)
        mine = json.loads(json.dumps(mine))
        assert mine == want, want["op"]


# The policy blocks of the reference's case files (configs/qwen_*.json, configs/llama_incremental.json),
# as the scheduler passes them on: CacheWindowSpec(**block), SlotPlacementSpec(**block).
QWEN_WINDOW = dict(allocation_bytes=448790528, allocation_count=80, bytes_per_token=2048, width_tokens=32768,
                   lookahead_tokens=16384, quantum_tokens=8192, min_update_seconds=1.0, idle_only=True)
LLAMA_WINDOW = dict(allocation_bytes=297795584, allocation_count=120, bytes_per_token=2048, width_tokens=21840,
                    lookahead_tokens=10920, quantum_tokens=5460, min_update_seconds=1.0, idle_only=True)
QWEN_SLOTS = dict(block_tokens=256, lookahead_tokens=4096, min_update_seconds=0.25, max_blocks_per_update=4,
                  active_seconds=2.0, refresh_seconds=10.0, max_feedback_lag_seconds=1.0)


def test_case_file_blocks_are_accepted(tmp_path, monkeypatch):
    for block in (QWEN_WINDOW, dict(QWEN_WINDOW, update_mode="full_cache"),
                  dict(QWEN_WINDOW, update_mode="initial_only"), LLAMA_WINDOW):
        spec = cw.CacheWindowSpec(**block)
        lo, hi = spec.window(0)
        assert (lo, hi) == (0, block["width_tokens"] * block["bytes_per_token"])
    # known answers at the two geometries (recorded from the reference)
    assert cw.CacheWindowSpec(**QWEN_WINDOW).window(16385) == (16777216, 83886080)
    assert cw.CacheWindowSpec(**QWEN_WINDOW).window(1e9) == (369098752, 436207616)
    assert cw.CacheWindowSpec(**LLAMA_WINDOW).window(10921) == (11182080, 55910400)
    assert cw.CacheWindowSpec(**LLAMA_WINDOW).window(145404) == (246005760, 290734080)
    monkeypatch.setenv("RETARGET_SLOT_FEEDBACK_DIR", str(tmp_path))
    ctl = sp.SlotPlacementController(cw.CacheWindowSpec(**QWEN_WINDOW), sp.SlotPlacementSpec(**QWEN_SLOTS), 4242)
    assert ctl.budget == 32768 // 256


def test_choose_random_snapshots_against_oracle():
    """The controller's ranking and selection on random snapshots -- ties in the
    stamps, blocks that are in both lists, stale and fresh commitments, changed
    versions -- against the oracle's restatement (itself pinned to the reference's
    logs in test_oracle_golden.py)."""
    import random

    from oracle import ref_policy as rp
    rng = random.Random(77)
    for _ in range(400):
        n_blocks = rng.choice([4, 16, 64])
        block_tokens = rng.choice([16, 256])
        budget = rng.randint(1, n_blocks)
        kw = dict(block_tokens=block_tokens, max_blocks_per_update=rng.randint(1, budget),
                  active_seconds=rng.choice([.5, 2.0]), refresh_seconds=rng.choice([1.0, 10.0]))
        ctl = sp.SlotPlacementController(
            cw.CacheWindowSpec(n_blocks * block_tokens * 2048, 2, 2048, budget * block_tokens, block_tokens // 2,
                               block_tokens // 2),
            sp.SlotPlacementSpec(**kw), 1, snapshot_source=lambda now: None)
        assert ctl.budget == budget
        now = 100.0
        stamp = lambda: now - rng.choice([0.0, .25, .5, 1.0, 2.0, 2.5, 30.0])
        snapshot = dict(
            recent_reads=[[b, stamp()] for b in rng.sample(range(n_blocks), rng.randint(0, n_blocks))],
            recent_writes=[[b, stamp()] for b in rng.sample(range(n_blocks), rng.randint(0, n_blocks // 2))],
            free_head_blocks=rng.sample(range(n_blocks), rng.randint(0, 3)),
            block_versions=[rng.randint(0, 2) for _ in range(n_blocks)])
        committed = {b: (rng.randint(0, 2), now - rng.choice([.1, 1.0, 5.0, 50.0]))
                     for b in rng.sample(range(n_blocks), rng.randint(0, n_blocks))}
        ctl.committed = dict(committed)
        want = rp.choose(snapshot, rp.SlotSpec(**kw), budget, committed, now)
        assert ctl.choose(snapshot, now) == want
        assert sp.target_blocks(snapshot, ctl.slot_spec, budget, now) == want[0]
