"""GPU parity for the device-resident slot-feedback state and its recency-ranked
plan, against the CPU restatement of the reference's event-driven chain
(SlotFeedback.consume/publish -> target_blocks -> choose -> blocksv) on the
incremental decode trace: arrivals, one token per live request per step,
finished requests returning pages to the free list.  Exact equality."""
import numpy as np
import pytest

from oracle import compose
from oracle import ref_policy as rp
from oracle import uvm_expand as ux
from retarget_b200 import capi, workloads
from retarget_b200.feedback import DeviceFeedback
from retarget_b200.planner import (DevicePlanner, ranges_from_tensor, ranges_to_tuples,
                                   result_from_tensor)

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def canonical(snapshot):
    s = dict(snapshot)
    for key in ("recent_reads", "recent_writes"):
        s[key] = sorted((-t, b) for b, t in s[key])
    for key in ("pid", "published_monotonic_s", "sequence"):   # host-side bookkeeping
        s.pop(key, None)
    return s


def run_trace(layout, trace, *, budget, max_blocks, active, refresh, evict, dt=0.03, clear_at=None,
              dtype=np.int64, fused=False):
    """`fused`: the step's three calls (alloc, attention, plan) as the one-launch
    `step()`; the oracle is driven the same either way."""
    dev = torch.device("cuda:0")
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    planner = DevicePlanner(layout, 0)
    fb = DeviceFeedback(planner, pid=0)
    spec = rp.SlotSpec(block_tokens=layout.block_tokens, max_blocks_per_update=max_blocks,
                       active_seconds=active, refresh_seconds=refresh)
    oracle = compose.FeedbackSession(layout, spec, budget, evict=evict)
    d_out = torch.zeros((1 << 14) * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    flags = capi.RT_PLAN_EVICT if evict else 0
    h = stream.cuda_stream
    moved = 0

    def up(ids):
        return torch.from_numpy(np.ascontiguousarray(ids).astype(dtype)).to(dev)

    for step, ev in enumerate(trace):
        t = 100.0 + step * dt
        if clear_at is not None and step == clear_at:
            fb.clear(t - 0.004, h)
            oracle.clear(t - 0.004)
        now = t + 0.001
        policy = dict(budget=budget, max_blocks_per_update=max_blocks, active_seconds=active,
                      refresh_seconds=refresh, flags=flags, d_out=d_out, d_result=d_res, stream=h)
        head = None if ev.free_head is None or not len(ev.alloc_slots) else up(ev.free_head)
        if fused:
            fb.step(d_allocated=up(ev.alloc_slots) if len(ev.alloc_slots) else None, t_allocated=t - 0.002,
                    d_free_head=head, d_read=up(ev.read_slots), d_written=up(ev.write_slots), t_attention=t,
                    now=now, **policy)
        else:
            if len(ev.alloc_slots):
                fb.alloc(up(ev.alloc_slots), t - 0.002, head, h)
            fb.attention(up(ev.read_slots), up(ev.write_slots), t, h)
            fb.plan(now, **policy)
        if len(ev.alloc_slots):
            oracle.alloc(ev.alloc_slots, ev.free_head, t - 0.002)
        oracle.attention(ev.read_slots, ev.write_slots, t)
        want, info = oracle.plan(now)
        torch.cuda.synchronize()
        res = result_from_tensor(d_res)
        got = ranges_to_tuples(ranges_from_tensor(d_out, res["n_ranges"]))
        assert got == want, f"step {step}: {info}"
        assert res["blocks_added"] == len(info["selected"]) and res["blocks_evicted"] == len(info["evicted"])
        assert planner.get_resident()[0] == info["committed"], f"step {step}"
        moved += len(want)
        if step % 16 == 0 or step == len(trace) - 1:
            assert canonical(fb.snapshot()) == canonical(oracle.snapshot()), f"step {step}"
    assert fb.arrays()[5] == 0
    fb.close()
    planner.close()
    return moved


FUSED = pytest.mark.parametrize("fused", [False, True], ids=["three-calls", "one-launch"])


@FUSED
def test_incremental_trace_config(fused):
    """40 layers, 65,536-slot pool, Poisson arrivals, 25 % budget, every step planned."""
    layout = workloads.Layout(40, 2048, 65536)
    trace = workloads.decode_trace(0, steps=256, initial_requests=12)
    moved = run_trace(layout, trace, budget=16, max_blocks=16, active=2.0, refresh=10.0, evict=True, fused=fused)
    assert moved > 0


@FUSED
@pytest.mark.parametrize("dtype", [np.int64, np.int32], ids=["i64", "i32"])
def test_reference_update_limits_refresh_and_allocator_clear(dtype, fused):
    """The reference's own policy values (4 new blocks per update), a short
    refresh period so that due-for-refresh blocks are re-sent, no eviction, and an
    allocator clear in the middle.  Once with 64-bit and once with 32-bit ids."""
    layout = workloads.Layout(4, 2048, 32768)
    trace = workloads.decode_trace(3, steps=120, pool_slots=32768, arrival_rate=1.0, median=256,
                                   mean_output=24, initial_requests=6)
    moved = run_trace(layout, trace, budget=8, max_blocks=4, active=2.0, refresh=0.5, evict=False,
                      clear_at=70, dtype=dtype, fused=fused)
    assert moved > 0


@FUSED
def test_small_blocks_wide_bitmap(fused):
    """1000 blocks of 6 slots: the multiply-shift division and a bitmap that
    fills every lane of the ranking kernel."""
    layout = workloads.Layout(2, 2048, 6001, 12288)
    trace = workloads.decode_trace(5, steps=60, pool_slots=5984, arrival_rate=0.7, median=200,
                                   mean_output=30, initial_requests=3)
    moved = run_trace(layout, trace, budget=300, max_blocks=300, active=0.2, refresh=5.0, evict=True,
                      fused=fused)
    assert moved > 0


def test_snapshot_feeds_the_python_controller():
    """SlotPlacementController driven by DeviceFeedback.snapshot picks the blocks
    the on-device plan picks."""
    from retarget_b200.cache_window import CacheWindowSpec
    from retarget_b200.slot_placement import SlotPlacementController, SlotPlacementSpec
    dev = torch.device("cuda:0")
    layout = workloads.Layout(2, 2048, 16384)
    planner = DevicePlanner(layout, 0)
    fb = DeviceFeedback(planner, pid=4242)
    slots = torch.tensor([5, 6, 7, 3000, 3001, 9000, 16000], dtype=torch.int64, device=dev)
    fb.alloc(slots, 10.0, torch.tensor([2048, 2049, 40], dtype=torch.int64, device=dev))
    fb.attention(slots[:5], slots[5:6], 10.5)
    ctl = SlotPlacementController(
        CacheWindowSpec(layout.alloc_bytes, layout.n_buffers, 2048, 4096, 1024, 1024),
        SlotPlacementSpec(block_tokens=1024, max_blocks_per_update=4), 4242, snapshot_source=fb.snapshot)
    snap = ctl.snapshot(10.6)
    assert snap["free_head_blocks"] == [2, 0] and snap["block_versions"][0] == 1
    desired, selected = ctl.choose(snap, 10.6)
    assert desired == [0, 2, 8, 15] and selected == [0, 2, 8, 15]
    fb.close()
    planner.close()


def test_published_file_feeds_the_controller(tmp_path, monkeypatch):
    """DeviceFeedback.publish writes <dir>/<pid>.json the way the reference's
    SlotFeedback does; a controller that reads the directory sees the same state."""
    import json
    import time
    from retarget_b200.cache_window import CacheWindowSpec
    from retarget_b200.slot_placement import SlotPlacementController, SlotPlacementSpec
    dev = torch.device("cuda:0")
    layout = workloads.Layout(2, 2048, 16384)
    planner = DevicePlanner(layout, 0)
    fb = DeviceFeedback(planner, pid=4242)
    now = time.monotonic()
    slots = torch.tensor([5, 6, 7, 3000, 3001, 9000, 16000], dtype=torch.int32, device=dev)
    fb.alloc(slots, now - 0.3, torch.tensor([2048, 2049, 40], dtype=torch.int32, device=dev))
    fb.attention(slots[:5], slots[5:6], now - 0.1)
    row = fb.publish(tmp_path)
    on_disk = json.loads((tmp_path / "4242.json").read_text())
    assert on_disk == row and not (tmp_path / ".4242.tmp").exists()
    assert on_disk["version"] == 1 and on_disk["block_tokens"] == 1024 and on_disk["epoch"] == 1
    monkeypatch.setenv("RETARGET_SLOT_FEEDBACK_DIR", str(tmp_path))
    ctl = SlotPlacementController(
        CacheWindowSpec(layout.alloc_bytes, layout.n_buffers, 2048, 4096, 1024, 1024),
        SlotPlacementSpec(block_tokens=1024, max_blocks_per_update=4), 4242)
    snap = ctl.snapshot(now)
    assert snap is not None and snap["free_head_blocks"] == [2, 0]
    assert ctl.choose(snap, now)[0] == [0, 2, 8, 15]
    fb.close()
    planner.close()


def test_device_writer_publishes_what_the_reference_probe_would(tmp_path):
    """DeviceWriter.submit fed with the decode trace as the probe's hooks would
    feed it (int32 kv indices, int64 written slots, free-head samples, a
    geometry event, frees, an allocator clear), against the restated
    SlotFeedback consuming the same rows as run lists: every file the writer
    drops equals the snapshot the reference would have published."""
    import json
    from retarget_b200.probe import DeviceWriter
    dev = torch.device("cuda:0")
    trace = workloads.decode_trace(7, steps=90, pool_slots=32768, arrival_rate=1.0, median=256,
                                   mean_output=24, initial_requests=6)
    capacity = 32767
    clock = {"t": 50.0}
    writer = DeviceWriter(tmp_path, pid=77, block_tokens=256, publish_seconds=.05, buffers=8, slot_bytes=2048,
                          clock=lambda: clock["t"])
    oracle = rp.FeedbackState(block_tokens=256, publish_seconds=.05, pid=77)
    sequence = 0
    published = 0

    def both(kind, tensors=None, **fields):
        nonlocal sequence, published
        if kind == "attention":
            sampled_out = clock["t"] - both.last_attention < .05
            if not sampled_out:
                both.last_attention = clock["t"]
        else:
            sampled_out = False
        writer.submit(kind, {k: (None if v is None else torch.from_numpy(v).to(dev)) for k, v in (tensors or {}).items()},
                      **fields)
        if sampled_out:
            return
        row = dict(event=kind, monotonic_s=clock["t"], sequence=sequence, **fields)
        sequence += 1
        for key, value in (tensors or {}).items():
            if value is not None:
                row[key + "_runs"] = rp.encode_runs(value.tolist())
        before = oracle.last_publish
        oracle.consume(row)
        if oracle.last_publish != before:
            published += 1
            on_disk = json.loads((tmp_path / "77.json").read_text())
            assert canonical(on_disk) == canonical(oracle.last_snapshot), (kind, sequence)
            assert on_disk["sequence"] == oracle.last_snapshot["sequence"]
            assert on_disk["observed_monotonic_s"] == oracle.last_snapshot["observed_monotonic_s"]
    both.last_attention = -float("inf")

    for step, ev in enumerate(trace):
        if step == 3:
            both("geometry", allocations=[dict(slot_bytes=2048)] * 8, allocator_size=capacity)
        if step == 60:
            both("allocator_clear", allocator_size=capacity, need_sort=False)
        if len(ev.alloc_slots):
            tensors = {"slot": ev.alloc_slots.astype(np.int64)}
            if ev.free_head is not None:
                tensors["free_head"] = ev.free_head.astype(np.int64)
            both("alloc", tensors, allocator_size=capacity, need_sort=False)
        clock["t"] += 0.011
        both("attention", {"read": ev.read_slots.astype(np.int32), "write": ev.write_slots.astype(np.int64)},
             path="eager", mode="DECODE", batch_size=ev.live, reads="all_cached_kv")
        clock["t"] += 0.011
        if step % 7 == 0 and len(ev.write_slots):
            both("free", {"slot": ev.write_slots[:1].astype(np.int64)}, grouped=False)
        clock["t"] += 0.011
    assert published > 20 and oracle.epoch == 2
    with pytest.raises(AssertionError):
        writer.submit("geometry", allocations=[dict(slot_bytes=4096)] * 8, allocator_size=capacity)
    writer.close()


def test_chain_over_the_recency_horizon():
    """The script recorded from the reference's whole chain (SlotFeedback ->
    snapshot file -> SlotPlacementController.update, 45 s): committed blocks that
    leave the desired set while nothing is selected stay on record and are not
    sent again when they return unchanged.  Device, oracle and the reference's
    recorded commands agree at every update."""
    import json
    from pathlib import Path
    from chain_replay import chain_session, replay_chain
    block = json.loads((Path(__file__).parent / "golden" / "reference_policy.json").read_text())["placement_chain"]
    session, layout = chain_session(block)
    dev = torch.device("cuda:0")
    planner = DevicePlanner(layout, 0)
    fb = DeviceFeedback(planner, pid=block["pid"])
    d_out = torch.zeros(4096 * 24, dtype=torch.uint8, device=dev)
    d_res = torch.zeros(64, dtype=torch.uint8, device=dev)
    up = lambda ids: torch.from_numpy(np.asarray(ids, dtype=np.int64)).to(dev)
    spec = session.spec

    def on_event(kind, f, t):
        if kind == "alloc":
            fb.alloc(up(f["slots"]), t, up(f["free_head"]) if "free_head" in f else None)
        elif kind == "attention":
            fb.attention(up(f["read"]), up(f["write"]), t)
        else:
            fb.free(t)

    def on_plan(t, want, info):
        fb.plan(t, budget=session.budget, max_blocks_per_update=spec.max_blocks_per_update,
                active_seconds=spec.active_seconds, refresh_seconds=spec.refresh_seconds, flags=0,
                d_out=d_out, d_result=d_res)
        torch.cuda.synchronize()
        res = result_from_tensor(d_res)
        assert ranges_to_tuples(ranges_from_tensor(d_out, res["n_ranges"])) == want, t
        assert planner.get_resident()[0] == info["committed"], t

    replay_chain(block, session, on_event=on_event, on_plan=on_plan)
    fb.close()
    planner.close()
