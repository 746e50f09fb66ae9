"""Replay of the script recorded from the reference's whole event-driven chain
(tests/golden/reference_policy.json, block "placement_chain") -- shared by the
CPU test of the oracle and the GPU test of the device-resident state."""
from oracle import ref_policy as rp


def replay_chain(block, session, *, on_event=None, on_plan=None):
    """Feeds the recorded script of the reference's whole event-driven chain to
    ``session`` (the oracle's FeedbackSession) and checks every controller update
    against what the reference sent and kept."""
    w = rp.WindowSpec(**block["cache_spec"])
    unit = session.spec.block_tokens * w.bytes_per_token
    for step in block["log"]:
        t, kind = step["t"], step["kind"]
        if kind != "update":
            f = step["fields"]
            if kind == "alloc":
                session.alloc(f["slots"], f.get("free_head"), t)
            elif kind == "attention":
                session.attention(f["read"], f["write"], t)
            else:
                session.free(f["slots"], t)
            if on_event:
                on_event(kind, f, t)
            continue
        out, info = session.plan(t)
        if on_plan:
            on_plan(t, out, info)
        if step["result"] is None:
            assert info["selected"] == [] and out == [], t
        else:
            assert info["desired"] == step["result"]["desired_blocks"], t
            assert info["selected"] == step["result"]["gpu_blocks"], t
            assert step["commands"] == [
                f"blocksv {block['generation']} {w.allocation_bytes} {w.allocation_count} {unit} "
                f"{rp.encode_mask(info['selected'])}"]
            assert sum(r[3] for r in out) == step["result"]["requested_gpu_bytes"]
        assert info["committed"] == step["committed"], t
        assert {str(k): v[0] for k, v in session.committed.items()} == step["committed_versions"], t


def chain_session(block):
    from oracle import compose
    from retarget_b200 import workloads
    w = rp.WindowSpec(**block["cache_spec"])
    s = rp.SlotSpec(**block["slot_spec"])
    layout = workloads.Layout(w.allocation_count // 2, w.bytes_per_token, block["capacity"] + 1,
                              s.block_tokens * w.bytes_per_token, True)
    assert layout.alloc_bytes == w.allocation_bytes and layout.n_buffers == w.allocation_count
    return compose.FeedbackSession(layout, s, rp.slot_plan_budget(w, s), evict=False), layout

