"""Range expansion pinned to the REAL reference library.

``tests/golden/reference_uvm_socket.json`` was recorded by ``oracle/drive_ref.py``:
the unmodified select.cpp, built and preloaded into a driver program under a
stub CUDA driver, answering 415 plan commands on its own control socket; each
entry holds the socket reply and the cuMemPrefetchAsync calls the plan caused.
Three implementations must reproduce it: the Python oracle, the C++ expander
behind ``rt_expand_command``, and this repository's UVM server + executor."""
import ctypes as C
import json
import os
from pathlib import Path

import pytest

from oracle import uvm_expand as ux

ROOT = Path(__file__).resolve().parent.parent
MIB = 1 << 20


@pytest.fixture(scope="module")
def recorded():
    return json.loads((ROOT / "tests" / "golden" / "reference_uvm_socket.json").read_text())


def chunked(ranges, chunk):
    out = []
    for rid, off, nbytes, dst in ranges:
        done = 0
        while done < nbytes:
            n = min(chunk, nbytes - done)
            out.append([rid, off + done, n, dst])
            done += n
    return out


def plan_lines(scenario):
    gen = None
    for r in scenario["results"]:
        if r["line"].strip() in ("status", "list"):
            gen = r["reply"].get("allocation_generation", gen)
            continue
        yield r


def generation_of(scenario):
    for r in scenario["results"]:
        if "allocation_generation" in r["reply"]:
            return r["reply"]["allocation_generation"]
    raise AssertionError("no status/list in the scenario")


def test_oracle_reproduces_the_reference_library(recorded):
    total = 0
    for sc in recorded["scenarios"]:
        gen, reg, chunk = generation_of(sc), sc["allocs"], sc["chunk_mb"] * MIB
        for r in plan_lines(sc):
            try:
                got, err = ux.command(reg, gen, r["line"]), None
            except ux.PlanError as e:
                got, err = None, str(e)
            if r["reply"].get("ok"):
                assert err is None, (r["line"], err)
                assert chunked(got, chunk) == r["calls"], r["line"]
                assert r["status"]["job_completed_bytes"] == sum(x[2] for x in got)
                assert r["status"]["last_error"] == 0
            else:
                assert err == r["reply"]["error"], r["line"]
            total += 1
    assert total > 400


def test_cpp_expander_reproduces_the_reference_library(recorded):
    from retarget_b200 import capi
    for sc in recorded["scenarios"]:
        gen, reg, chunk = generation_of(sc), sc["allocs"], sc["chunk_mb"] * MIB
        for r in plan_lines(sc):
            got, err = capi.expand_command(reg, gen, r["line"])
            if r["reply"].get("ok"):
                assert err is None, (r["line"], err)
                assert chunked([list(x) for x in got], chunk) == r["calls"], r["line"]
            else:
                assert err == r["reply"]["error"], r["line"]


def test_list_and_status_replies_match(recorded):
    sc = recorded["scenarios"][0]
    listing = next(r for r in sc["results"] if r["line"] == "list")["reply"]
    assert listing["allocations"] == [{"id": a["id"], "bytes": a["bytes"], "device": 0} for a in sc["allocs"]]
    sc2 = recorded["scenarios"][1]
    listing = next(r for r in sc2["results"] if r["line"] == "list")["reply"]
    assert [a["id"] for a in listing["allocations"]] == [1, 3, 4, 5] and listing["allocation_generation"] == 6


def test_this_repositorys_preload_library_gives_the_same_answers(recorded):
    """The same driver program, the same stub driver, our LD_PRELOAD library
    instead of the reference's: same replies and the same prefetch calls (ours
    may order the calls of one phase differently across its streams, so calls are
    compared as CPU-phase and GPU-phase multisets, CPU phase first)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("drive_ref", ROOT / "oracle" / "drive_ref.py")
    drive = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(drive)
    import subprocess
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "_ref/stubs/libcuda.so", "_ref/drive_app"], check=True,
                   capture_output=True)
    ours = ROOT / "retarget_b200" / "libretarget_preload.so"
    if not ours.exists():
        pytest.skip("preload library not built")
    for sc in recorded["scenarios"]:
        got = drive.run(ours, sc["sizes"], [r["line"] for r in sc["results"]], sc["chunk_mb"])
        assert got["allocs"] == sc["allocs"]
        for mine, ref in zip(got["results"], sc["results"]):
            line = ref["line"]
            if line.strip() in ("status", "list"):
                keep = ("ok", "managed_bytes", "allocation_count", "allocation_generation", "allocations", "busy")
                assert {k: mine["reply"].get(k) for k in keep} == {k: ref["reply"].get(k) for k in keep}, line
                continue
            assert mine["reply"].get("ok") == ref["reply"].get("ok"), line
            if not ref["reply"].get("ok"):
                assert mine["reply"] == ref["reply"], line
                continue
            assert mine["reply"]["job_id"] == ref["reply"]["job_id"], line
            for key in ("job_completed_bytes", "last_error", "completed_job", "completed_cpu_bytes",
                        "completed_gpu_bytes"):
                assert mine["status"][key] == ref["status"][key], (line, key)
            cpu_m = sorted(c for c in mine["calls"] if c[3] < 0)
            cpu_r = sorted(c for c in ref["calls"] if c[3] < 0)
            assert cpu_m == cpu_r, line
            assert sorted(c for c in mine["calls"] if c[3] >= 0) == sorted(c for c in ref["calls"] if c[3] >= 0), line
            kinds = [c[3] >= 0 for c in mine["calls"]]
            assert kinds == sorted(kinds), line                      # every CPU-bound call first
