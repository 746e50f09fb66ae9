"""The LD_PRELOAD library under a stub driver: an application that looks the
driver up with dlopen/dlsym/cuGetProcAddress gets its device allocations turned
into registered managed allocations, and can be driven through the control
socket of its own process."""
import json
import os
import subprocess
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
PRELOAD = ROOT / "retarget_b200" / "libretarget_preload.so"
FAKE = HERE / "fake_cuda" / "libcuda_fake.so"


def run_app(extra_env, *args):
    from test_uvm_server import build_fake
    build_fake()
    app = HERE / "fake_cuda" / "preload_app"
    src = HERE / "fake_cuda" / "preload_app.c"
    if not app.exists() or app.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O1", "-o", str(app), str(src), "-ldl"], check=True)
    env = dict(os.environ, RETARGET_B200_LIBCUDA=str(FAKE), LD_PRELOAD=str(PRELOAD), **extra_env)
    out = subprocess.run([str(app), str(FAKE), *args], env=env, capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    return out.stdout


def replies(text):
    out = {}
    for line in text.splitlines():
        if line.startswith("REPLY "):
            cmd, _, body = line[6:].partition(" -> ")
            out.setdefault(cmd.split()[0], []).append(json.loads(body))
    return out


@pytest.mark.skipif(not PRELOAD.exists(), reason="preload library not built")
def test_allocations_are_converted_registered_and_planned():
    text = run_app({"SELECT_UVM_ENABLE": "1", "SELECT_UVM_CONVERT_ALLOC": "1"}, "fork")
    r = replies(text)
    first, after = r["list"]
    assert first["allocation_generation"] == 5
    assert [a["bytes"] for a in first["allocations"]] == [32 << 20] * 4 + [4096]
    assert r["windowv"][0] == {"ok": True, "job_id": 1}
    done = r["status"][1]
    assert done["completed_job"] == 1 and done["last_error"] == 0
    assert done["completed_cpu_bytes"] == 4 * (24 << 20)
    assert done["completed_gpu_bytes"] == 4 * (8 << 20) + 4096     # window + the non-cache allocation
    # cuMemFree resolved through cuGetProcAddress is hooked as well
    assert after["allocation_generation"] == 6 and [a["id"] for a in after["allocations"]] == [1, 3, 4, 5]
    log = text.split("DRIVER LOG\n")[1].splitlines()
    assert sum(l.startswith("alloc_managed") for l in log) == 5 and not any(l.startswith("alloc_device") for l in log)
    kinds = [int(l.split()[3]) for l in log if l.startswith("prefetch")]
    assert kinds == sorted(kinds)                                   # every CPU-bound call first
    assert "child alloc=3" in text                                  # a forked child may not use CUDA


@pytest.mark.skipif(not PRELOAD.exists(), reason="preload library not built")
def test_disabled_library_is_transparent():
    text = run_app({})
    log = text.split("DRIVER LOG\n")[1].splitlines()
    assert sum(l.startswith("alloc_device") for l in log) == 5
    assert "connect failed" in text
