"""Host side under sanitizers: the UVM server, plan expansion and driver table
are compiled together with a stress program (tests/stress/uvm_stress.cpp) once
with ThreadSanitizer and once with AddressSanitizer + UBSan, and run against the
stub driver; the worker pool of the id narrowing gets the same treatment
(tests/stress/pack_stress.cpp).  The reference has no race detection at all; its concurrency is a
lock-order convention (select.cpp:23750-23754), which is what the stress
exercises: allocation hooks, two socket clients, an in-process submitter and
stop/start cycles, all at once."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

from test_uvm_server import build_fake

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
CSRC = ROOT / "retarget_b200" / "csrc"
OUT = HERE / "stress" / "_build"
SOURCES = [CSRC / "host_policy.cpp", CSRC / "uvm_plan.cpp", CSRC / "uvm_server.cpp",
           CSRC / "driver_api.cpp", HERE / "stress" / "uvm_stress.cpp"]


def cuda_include():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return str(Path(nvcc).resolve().parent.parent / "include")


PACK_SOURCES = [CSRC / "host_pack.cpp", HERE / "stress" / "pack_stress.cpp"]


def build(name, flags, sources=SOURCES, stem="uvm_stress"):
    OUT.mkdir(parents=True, exist_ok=True)
    exe = OUT / f"{stem}_{name}"
    deps = sources + list(CSRC.glob("*.h")) + [ROOT / "include" / "retarget_b200.h"]
    if not exe.exists() or any(d.stat().st_mtime > exe.stat().st_mtime for d in deps):
        subprocess.run(["g++", "-O1", "-g", "-fno-omit-frame-pointer", "-std=c++17", "-pthread", *flags,
                        f"-I{ROOT / 'include'}", f"-I{CSRC}", f"-I{cuda_include()}",
                        *map(str, sources), "-o", str(exe), "-ldl", "-lrt"], check=True)
    return exe


SANITIZERS = pytest.mark.parametrize("name,flags,env", [
    ("tsan", ["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=0 exitcode=66"}),
    ("asan", ["-fsanitize=address,undefined"], {"ASAN_OPTIONS": "detect_leaks=1",
                                                "UBSAN_OPTIONS": "halt_on_error=1 print_stacktrace=1"}),
])


@SANITIZERS
def test_id_narrowing_pool_under_sanitizer(name, flags, env):
    """Three threads share the worker pool of the host-buffer call's id narrowing."""
    exe = build(name, flags, PACK_SOURCES, "pack_stress")
    proc = subprocess.run([str(exe), "12"], capture_output=True, text=True, env={**os.environ, **env}, timeout=300)
    out = proc.stdout + proc.stderr
    if "unexpected memory mapping" in out or "Shadow memory range interleaves" in out:
        pytest.skip("the sanitizer runtime cannot map its shadow memory on this host")
    assert proc.returncode == 0, out[-6000:]
    assert "WARNING: ThreadSanitizer" not in out and "ERROR: AddressSanitizer" not in out, out[-6000:]
    assert "runtime error" not in out and "bad=0" in out, out[-6000:]


@SANITIZERS
def test_uvm_server_stress_under_sanitizer(name, flags, env, tmp_path):
    exe = build(name, flags)
    sock = tmp_path / "ctl.sock"
    proc = subprocess.run([str(exe), str(build_fake()), str(sock), "2"], capture_output=True, text=True,
                          env={**os.environ, **env}, timeout=120)
    out = proc.stdout + proc.stderr
    if "unexpected memory mapping" in out or "Shadow memory range interleaves" in out:
        pytest.skip("the sanitizer runtime cannot map its shadow memory on this host")
    assert proc.returncode == 0, out[-6000:]
    assert "WARNING: ThreadSanitizer" not in out and "ERROR: AddressSanitizer" not in out, out[-6000:]
    assert "runtime error" not in out, out[-6000:]
    assert " bad=0" in out and not sock.exists()
