"""UVM control server + prefetch executor on a CPU-only host: the library's
driver table is pointed at a stub driver that logs every call.  Checks the
socket protocol (replies, error strings, ordering rules) and that each accepted
plan turns into exactly the prefetch calls the oracle's range list implies."""
import ctypes as C
import json
import os
import socket
import subprocess
import threading
import time
from pathlib import Path

import pytest

from oracle import uvm_expand as ux

HERE = Path(__file__).resolve().parent
FAKE = HERE / "fake_cuda" / "libcuda_fake.so"
MIB = 1 << 20


def build_fake():
    src = HERE / "fake_cuda" / "fake_cuda.c"
    if not FAKE.exists() or FAKE.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O1", "-shared", "-fPIC", "-o", str(FAKE), str(src), "-ldl", "-lpthread"],
                       check=True)
    return FAKE


from retarget_b200.capi import UvmConfig as RtUvmConfig  # noqa: E402


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    os.environ["RETARGET_B200_LIBCUDA"] = str(build_fake())
    from retarget_b200 import capi
    from retarget_b200.control import LocalUvm, UvmController
    lib = capi.lib
    fake = C.CDLL(str(FAKE), mode=C.RTLD_GLOBAL)
    fake.fake_cuda_log.restype = C.c_size_t
    lib.rt_uvm_register.argtypes = [C.c_uint64, C.c_uint64, C.c_void_p, C.c_int, C.c_int,
                                    C.POINTER(C.c_uint64)]
    lib.rt_uvm_unregister_ptr.argtypes = [C.c_uint64]
    lib.rt_uvm_wait.argtypes = [C.c_uint64, C.c_double, C.POINTER(C.c_int)]
    sock = str(tmp_path_factory.mktemp("uvm") / "ctl.sock")
    cfg = RtUvmConfig(sock.encode(), 16 * MIB, 64 * MIB, 3, 1)
    assert lib.rt_uvm_start(C.byref(cfg)) == 0

    class Env:
        pass
    env = Env()
    env.lib, env.fake, env.sock = lib, fake, sock
    env.local = LocalUvm()
    env.remote = UvmController(os.getpid(), path=sock)
    env.registry = []          # mirrors the server's registry for the oracle

    def register(nbytes, ptr, device=0, concurrent=1):
        out = C.c_uint64()
        assert lib.rt_uvm_register(ptr, nbytes, None, device, concurrent, C.byref(out)) == 0
        env.registry.append(dict(id=out.value, bytes=nbytes, device=device, concurrent=concurrent, ptr=ptr))
        return out.value

    def log():
        buf = C.create_string_buffer(1 << 20)
        fake.fake_cuda_log(buf, len(buf))
        return buf.value.decode().splitlines()
    env.register, env.log = register, log
    yield env
    assert lib.rt_uvm_stop() == 0
    assert not os.path.exists(sock)          # the server removes the socket it created


def run_plan(env, line, via="local"):
    """Sends a plan, waits for the job, returns (reply, prefetch calls)."""
    env.fake.fake_cuda_reset()
    client = env.local if via == "local" else env.remote
    reply = client.command(line)
    if reply.get("ok"):
        client._wait_job(reply["job_id"], timeout=10, poll_seconds=0.002)
    calls = [tuple(l.split()[1:4]) for l in env.log() if l.startswith("prefetch")]
    return reply, [(int(p, 16), int(b), int(d)) for p, b, d in calls]


def expected_calls(env, ranges, chunk=16 * MIB):
    ptr = {a["id"]: a["ptr"] for a in env.registry}
    out = []
    for rid, off, nbytes, dst in ranges:
        done = 0
        while done < nbytes:
            n = min(chunk, nbytes - done)
            out.append((ptr[rid] + off + done, n, dst))
            done += n
    return out


def test_status_and_list_replies(server):
    env = server
    assert env.local.command("status") == env.remote.command("status")
    st = env.local.status()
    assert (st.pid, st.allocation_count, st.busy, st.job_id) == (os.getpid(), 0, False, 0)
    base = 0x7e0000000000
    for k in range(4):
        env.register(128 * MIB, base + k * (1 << 30))
    env.register(1 * MIB, base + (1 << 36))
    env.register(12345 * 4096, base + (1 << 37), device=0)
    gen, allocs = env.remote._allocation_snapshot()
    assert gen == 6 and [a["id"] for a in allocs] == [1, 2, 3, 4, 5, 6]
    assert allocs[0] == {"id": 1, "bytes": 128 * MIB, "device": 0}
    st = env.remote.status()
    assert st.managed_bytes == 4 * 128 * MIB + MIB + 12345 * 4096 and st.allocation_generation == 6
    # byte-exact reply text of `list`
    raw = C.create_string_buffer(4096)
    n = env.lib.rt_uvm_command(b"list", raw, 4096)
    assert raw.raw[:n].decode().startswith(
        '{"ok":true,"allocation_generation":6,"allocations":[{"id":1,"bytes":134217728,"device":0},')


@pytest.mark.parametrize("via", ["local", "socket"])
def test_plans_become_the_oracles_prefetch_calls(server, via):
    env = server
    gen = env.local.status().allocation_generation
    A = 128 * MIB
    lines = [
        f"windowv {gen} {A} 4 {ux.UINT64_MAX} {ux.UINT64_MAX} 0 {32 * MIB}",
        f"windowv {gen} {A} 4 0 {32 * MIB} {2 * MIB} {34 * MIB}",
        f"windowfullv {gen} {A} 4 {2 * MIB} {34 * MIB} {64 * MIB} {A}",
        f"blocksv {gen} {A} 4 {2 * MIB} f00f1",
        f"prefetch 5 0 {MIB} cpu",
        f"target {100 * MIB}",
        f"retarget {gen} {100 * MIB} {300 * MIB}",
        f"targetv {gen} 0",
    ]
    for line in lines:
        want = ux.command(env.registry, gen, line)
        reply, calls = run_plan(env, line, via)
        assert reply.get("ok"), (line, reply)
        assert calls == expected_calls(env, want), line
        st = env.local.status()
        assert st.last_error == 0 and st.completed_job == reply["job_id"]
        assert st.job_completed_bytes == sum(r[2] for r in want)


def test_cpu_phase_is_waited_for_before_the_gpu_phase(server):
    env = server
    gen = env.local.status().allocation_generation
    env.fake.fake_cuda_reset()
    reply = env.local.command(f"windowv {gen} {128 * MIB} 4 0 {32 * MIB} {16 * MIB} {48 * MIB}")
    env.local._wait_job(reply["job_id"], timeout=10, poll_seconds=0.002)
    events = [l.split() for l in env.log() if l.startswith(("prefetch", "sync"))]
    dsts = [int(e[3]) if e[0] == "prefetch" else None for e in events]
    first_gpu = next(i for i, d in enumerate(dsts) if d is not None and d >= 0)
    last_cpu = max(i for i, d in enumerate(dsts) if d == -1)
    assert last_cpu < first_gpu
    assert any(e[0] == "sync" for e in events[last_cpu:first_gpu])
    # streams are created once and reused: none is created by later jobs
    env.fake.fake_cuda_reset()
    reply = env.local.command(f"prefetch 5 0 {MIB} gpu")
    env.local._wait_job(reply["job_id"], timeout=10, poll_seconds=0.002)
    assert not [l for l in env.log() if l.startswith(("stream_create", "stream_destroy"))]


def test_rejections_use_the_socket_error_strings(server):
    env = server
    gen = env.local.status().allocation_generation
    A = 128 * MIB
    cases = [
        ("bogus", "invalid_command"),
        (f"windowv {gen + 1} {A} 4 0 0 0 {MIB}", "stale_allocations"),
        (f"windowv {gen} {A} 3 0 0 0 {MIB}", "cache_allocation_count_mismatch"),
        (f"windowv {gen} {A} 4 0 0 5 {MIB}", "invalid_window"),
        (f"blocksv {gen} {A} 4 {2 * MIB} 0", "empty_block_mask"),
        (f"blocksv {gen} {A} 4 {2 * MIB} 1{'0' * 16}", "block_out_of_range"),
        (f"blocksv {gen} {A} 4 {2 * MIB} xyz", "invalid_block_mask"),
        (f"blocksv {gen} {A} 4 123 1", "invalid_block_geometry"),
        ("prefetch 99 0 4096 gpu", "unknown_id"),
        ("prefetch 5 4096 0 gpu", "invalid_range"),
        ("prefetch 5 100 4096 gpu", "unaligned_range"),
        (f"target {1 << 50}", "target_exceeds_managed_bytes"),
        ("target 100", "unaligned_target"),
    ]
    for line, error in cases:
        for client in (env.local, env.remote):
            assert client.command(line) == {"ok": False, "error": error}, line
    for line, error in cases[1:]:
        with pytest.raises(ux.PlanError) as e:
            ux.command(env.registry, gen, line)
        assert str(e.value) == error
    assert env.local.status().busy is False


def test_raw_socket_line_rules(server):
    env = server

    def raw(payload: bytes):
        with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as s:
            s.settimeout(3)
            s.connect(env.sock)
            s.sendall(payload)
            data = b""
            while not data.endswith(b"\n"):
                chunk = s.recv(4096)
                if not chunk:
                    break
                data += chunk
            return json.loads(data)
    assert raw(b"status\n")["ok"] is True
    assert raw(b"a" * 600 + b"\n") == {"ok": False, "error": "invalid_line"}
    assert raw(b"sta\0tus\n") == {"ok": False, "error": "invalid_line"}
    assert raw(b"1 2 3 4 5 6 7 8 9\n") == {"ok": False, "error": "invalid_command"}
    t0 = time.time()
    assert raw(b"status") == {"ok": False, "error": "invalid_line"}     # no newline: 1 s timeout
    assert 0.5 < time.time() - t0 < 3
    assert os.stat(env.sock).st_mode & 0o777 == 0o600


def test_busy_and_error_latching(server):
    env = server
    gen = env.local.status().allocation_generation
    env.fake.fake_cuda_reset()
    env.fake.fake_cuda_set_sync_delay_us(300000)
    first = env.local.command(f"prefetch 1 0 {64 * MIB} gpu")
    assert first["ok"]
    assert env.local.command(f"prefetch 1 0 {MIB} gpu") == {"ok": False, "error": "busy"}
    assert env.local.status().busy is True                  # status never waits for the migration
    env.local._wait_job(first["job_id"], timeout=10, poll_seconds=0.01)
    # a failing driver call aborts the job and is latched in status
    env.fake.fake_cuda_reset()
    env.fake.fake_cuda_fail_prefetch(2, 719)
    reply = env.local.command(f"blocksv {gen} {128 * MIB} 4 {2 * MIB} ff")
    from retarget_b200.control import ControlError
    with pytest.raises(ControlError, match="CUDA error 719"):
        env.local._wait_job(reply["job_id"], timeout=10, poll_seconds=0.002)
    assert env.local.status().last_error == 719
    calls = [l for l in env.log() if l.startswith("prefetch")]
    assert len(calls) == 3                                   # nothing issued after the failure
    # the next accepted job clears the latch
    ok = env.local.command(f"prefetch 5 0 {MIB} gpu")
    env.local._wait_job(ok["job_id"], timeout=10, poll_seconds=0.002)
    assert env.local.status().last_error == 0


def test_generation_moves_with_the_registry(server):
    env = server
    gen = env.local.status().allocation_generation
    line = f"blocksv {gen} {128 * MIB} 4 {2 * MIB} 1"
    new_id = env.register(4096, 0x7d0000000000, concurrent=0)
    assert env.local.command(line) == {"ok": False, "error": "stale_allocations"}
    assert env.local.command(f"prefetch {new_id} 0 4096 gpu") == {
        "ok": False, "error": "concurrent_managed_access_required"}
    assert env.lib.rt_uvm_unregister_ptr(0x7d0000000000) == 1
    env.registry.pop()
    assert env.local.status().allocation_generation == gen + 2
    reply, calls = run_plan(env, f"blocksv {gen + 2} {128 * MIB} 4 {2 * MIB} 1")
    assert reply["ok"] and len(calls) == 4


@pytest.mark.parametrize("via", ["local", "socket"])
def test_prefix_plans_through_the_client(server, via):
    """set_target / retarget of the client against the running server: the
    prefetch calls are the oracle's expansion of targetv / retarget for the
    page-aligned targets, and an incremental retarget moves only the difference."""
    from retarget_b200.control import UvmRetargetResult, UvmTargetResult, aligned_uvm_target
    env = server
    client = env.local if via == "local" else env.remote
    client._placed = None
    sizes = [a["bytes"] for a in env.registry]
    page = os.sysconf("SC_PAGE_SIZE")

    def calls_of(action):
        env.fake.fake_cuda_reset()
        result = action()
        calls = [tuple(l.split()[1:4]) for l in env.log() if l.startswith("prefetch")]
        return result, [(int(p, 16), int(b), int(d)) for p, b, d in calls]

    gen = env.local.status().allocation_generation
    first = 200 * MIB + 1234
    res, calls = calls_of(lambda: client.set_target(first))
    t1 = aligned_uvm_target(sizes, first, page)
    assert isinstance(res, UvmTargetResult) and res.submitted_bytes == t1 and res.clamped_bytes == first
    assert calls == expected_calls(env, ux.expand_target(env.registry, gen, nbytes=t1, gen=gen))
    second = 330 * MIB + 4099
    res, calls = calls_of(lambda: client.retarget(first, second))
    t2 = aligned_uvm_target(sizes, second, page)
    assert isinstance(res, UvmRetargetResult) and (res.previous_submitted_bytes, res.submitted_bytes) == (t1, t2)
    assert calls == expected_calls(env, ux.expand_retarget(env.registry, gen, gen=gen, old=t1, new=t2))
    assert sum(c[1] for c in calls) == t2 - t1
    # a previous target the client did not submit: full plan instead
    res, calls = calls_of(lambda: client.retarget(17 * MIB, 64 * MIB))
    assert isinstance(res, UvmTargetResult)
    assert calls == expected_calls(env, ux.expand_target(env.registry, gen, nbytes=64 * MIB, gen=gen))
    # submitted without waiting, settled by wait_idle, then shrunk incrementally
    job = client.set_target(10 ** 12, wait=False)
    assert isinstance(job, int) and client._pending_job == job
    st = client.wait_idle(timeout=20)
    assert client._pending_job is None and client._submitted_target == st.managed_bytes
    res, calls = calls_of(lambda: client.retarget(10 ** 12, 0))
    assert isinstance(res, UvmRetargetResult) and sum(c[1] for c in calls) == st.managed_bytes
    assert all(c[2] == ux.CPU for c in calls)


def test_device_planner_ranges_can_be_submitted_directly(server):
    """rt_uvm_submit_ranges: planner output -> job, without the text round trip."""
    import numpy as np
    from retarget_b200 import capi
    env = server
    ranges = np.zeros(3, dtype=capi.RANGE_DTYPE)
    ranges[0] = (1, -1, 0, 2 * MIB)
    ranges[1] = (0, 0, 4 * MIB, 40 * MIB)
    ranges[2] = (3, 0, 126 * MIB, 2 * MIB)
    ids = (C.c_uint64 * 4)(1, 2, 3, 4)
    job = C.c_uint64()
    env.fake.fake_cuda_reset()
    env.lib.rt_uvm_submit_ranges.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t,
                                             C.POINTER(C.c_uint64)]
    assert env.lib.rt_uvm_submit_ranges(ranges.ctypes.data, 3, ids, 4, C.byref(job)) == 0
    err = C.c_int(-1)
    assert env.lib.rt_uvm_wait(job.value, 10.0, C.byref(err)) == 0 and err.value == 0
    calls = [(int(p, 16), int(b), int(d)) for p, b, d in
             (l.split()[1:4] for l in env.log() if l.startswith("prefetch"))]
    want = [(2, 0, 2 * MIB, -1), (1, 4 * MIB, 40 * MIB, 0), (4, 126 * MIB, 2 * MIB, 0)]
    assert calls == expected_calls(env, want)
    bad = ranges.copy()
    bad[1] = (0, 0, 4 * MIB, 200 * MIB)
    assert env.lib.rt_uvm_submit_ranges(bad.ctypes.data, 3, ids, 4, C.byref(job)) == -1


def test_side_streams_are_tracked_per_device(server):
    """Dropping one device's records leaves the other contexts' side streams in
    place: the next job on them creates no new streams, and none are destroyed
    that belong to a context the caller says is gone."""
    env = server
    ctx0, ctx1 = 0xC000, 0xC001                  # the stub driver's primary contexts of devices 0 and 1

    def register(ptr, ctx, device):
        out = C.c_uint64()
        assert env.lib.rt_uvm_register(ptr, 4 * MIB, C.c_void_p(ctx), device, 1, C.byref(out)) == 0
        return out.value

    def prefetch(rid):
        env.fake.fake_cuda_reset()
        reply = env.local.command(f"prefetch {rid} 0 {4 * MIB} gpu")
        assert reply["ok"], reply
        env.local._wait_job(reply["job_id"], timeout=10, poll_seconds=0.002)
        lines = env.log()
        return sum(l.startswith("stream_create") for l in lines), sum(l.startswith("stream_destroy") for l in lines)

    a = register(0x7f1000000000, ctx0, 0)
    b = register(0x7f2000000000, ctx1, 1)
    assert prefetch(a) == (3, 0) and prefetch(b) == (3, 0)       # three side streams per context, made on first use
    assert prefetch(a) == (0, 0)                                 # ... and kept
    env.lib.rt_uvm_unregister_device.argtypes = [C.c_int]
    env.fake.fake_cuda_reset()
    assert env.lib.rt_uvm_unregister_device(1) == 1
    assert not any(l.startswith("stream_destroy") for l in env.log())     # that context is gone: handles dropped
    b2 = register(0x7f3000000000, ctx1, 1)
    assert prefetch(a) == (0, 0)                                 # device 0 kept its streams
    assert prefetch(b2) == (3, 0)                                # device 1 starts over
    for ptr in (0x7f1000000000, 0x7f3000000000):
        assert env.lib.rt_uvm_unregister_ptr(ptr) == 1


def test_overlapped_phases_move_both_ways_at_once(server):
    """With `overlap_phases` the CPU-bound and the GPU-bound stretch of a plan are
    issued in turn inside one batch (no wait between them), each on its own side
    streams; the same chunks are prefetched, the same bytes are accounted."""
    env = server
    base = 0x7f4000000000
    ids = [env.register(128 * MIB, base + k * (1 << 30)) for k in range(4)]
    gen = env.local.status().allocation_generation
    n_alloc = sum(1 for a in env.registry if a["bytes"] == 128 * MIB)
    line = f"windowv {gen} {128 * MIB} {n_alloc} 0 {32 * MIB} {16 * MIB} {48 * MIB}"

    def run():
        env.fake.fake_cuda_reset()
        reply = env.local.command(line)
        assert reply["ok"], reply
        done = env.local._wait_job(reply["job_id"], timeout=10, poll_seconds=0.002)
        events = [l.split() for l in env.log() if l.startswith(("prefetch", "sync"))]
        return events, done

    in_order, done_a = run()
    assert env.lib.rt_uvm_stop() == 0
    cfg = RtUvmConfig(env.sock.encode(), 16 * MIB, 64 * MIB, 4, 1, 1)
    assert env.lib.rt_uvm_start(C.byref(cfg)) == 0
    try:
        overlapped, done_b = run()
    finally:
        assert env.lib.rt_uvm_stop() == 0
        cfg = RtUvmConfig(env.sock.encode(), 16 * MIB, 64 * MIB, 3, 1)
        assert env.lib.rt_uvm_start(C.byref(cfg)) == 0
    chunks = lambda events: sorted((e[1], int(e[2]), int(e[3])) for e in events if e[0] == "prefetch")
    assert chunks(in_order) == chunks(overlapped) and done_a.job_completed_bytes == done_b.job_completed_bytes
    # the reference's order waits between the phases; the overlapped one alternates directions before any wait
    first_sync = next(i for i, e in enumerate(overlapped) if e[0] == "sync")
    before = [int(e[3]) for e in overlapped[:first_sync]]
    assert -1 in before and any(d >= 0 for d in before)
    assert any(a != b for a, b in zip(before, before[1:]))
    # each direction keeps to its own streams
    streams = {}
    for e in overlapped:
        if e[0] == "prefetch":
            streams.setdefault(int(e[3]) < 0, set()).add(e[4])
    assert not (streams[True] & streams[False])
    for k in range(4):
        assert env.lib.rt_uvm_unregister_ptr(base + k * (1 << 30)) == 1
    env.registry[:] = [a for a in env.registry if a["id"] not in ids]
