"""Builds the native libraries in-tree with nvcc / g++ (sm_100a only).

    python -m retarget_b200.build            # build what is out of date
    python -m retarget_b200.build --force

Outputs (next to this file, ignored by git):
    libretarget_b200.so     C ABI: planner kernels, host policy, UVM server
    libretarget_preload.so  LD_PRELOAD library: driver-API hooks around the same server
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"
OBJ = ROOT / "build" / "obj"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-Wall", f"-I{INCLUDE}", f"-I{CSRC}"]
CXX_FLAGS = ["-O2", "-g", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-pthread",
             f"-I{INCLUDE}", f"-I{CSRC}"]

CORE_CU = ["plan_kernels.cu", "plan_capi.cu"]
CORE_CPP = ["host_policy.cpp", "uvm_plan.cpp", "controllers.cpp", "uvm_client.cpp", "host_pack.cpp"]
OPTIONAL_CORE_CPP = ["uvm_server.cpp", "driver_api.cpp"]
OPTIONAL_CORE_CU = ["feedback_kernels.cu", "paged_reader.cu", "paged_attention.cu", "noalloc_scan.cu", "read_probe.cu"]
PRELOAD_CPP = ["preload_hooks.cpp"]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA toolkit is required to build retarget_b200")


def cuda_include() -> str:
    return str(Path(nvcc()).resolve().parent.parent / "include")


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode:
        sys.stderr.write(" ".join(map(str, cmd)) + "\n" + proc.stdout + proc.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} {cmd[-1]}")
    return proc.stdout + proc.stderr


def build(force: bool = False, verbose: bool = False) -> dict:
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    objs = []
    log = []
    compiled = []                # what this call had to (re)make: empty when everything was up to date
    cu = CORE_CU + [f for f in OPTIONAL_CORE_CU if (CSRC / f).exists()]
    cpp = CORE_CPP + [f for f in OPTIONAL_CORE_CPP if (CSRC / f).exists()]
    for name in cu:
        src, obj = CSRC / name, OBJ / (name + ".o")
        if force or _stale(obj, [src, *headers]):
            log.append(_run([nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []),
                             "-c", str(src), "-o", str(obj)]))
            compiled.append(name)
        objs.append(obj)
    for name in cpp:
        src, obj = CSRC / name, OBJ / (name + ".o")
        if force or _stale(obj, [src, *headers]):
            log.append(_run(["g++", *CXX_FLAGS, f"-I{cuda_include()}", "-c", str(src), "-o", str(obj)]))
            compiled.append(name)
        objs.append(obj)
    core = PKG / "libretarget_b200.so"
    if force or _stale(core, objs):
        _run([nvcc(), "-shared", "-o", str(core), *map(str, objs),
              "-cudart", "static", "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"])
        compiled.append(core.name)
    out = {"core": core}
    pre_srcs = [CSRC / f for f in PRELOAD_CPP if (CSRC / f).exists()]
    if pre_srcs:
        pre_objs = []
        for src in pre_srcs:
            obj = OBJ / (src.name + ".o")
            if force or _stale(obj, [src, *headers]):
                _run(["g++", *CXX_FLAGS, f"-I{cuda_include()}", "-c", str(src), "-o", str(obj)])
                compiled.append(src.name)
            pre_objs.append(obj)
        pre = PKG / "libretarget_preload.so"
        if force or _stale(pre, pre_objs + objs):
            _run([nvcc(), "-shared", "-o", str(pre), *map(str, pre_objs), *map(str, objs),
                  "-cudart", "static", "-lpthread", "-ldl", "-lrt"])
            compiled.append(pre.name)
        out["preload"] = pre
    if verbose:
        print("".join(log))
    out["compiled"] = compiled
    return out


def build_stall_variant(force: bool = False) -> Path:
    """Test build of the core library in which the bulk-copy kernel's producer
    skips one copy and the bounded waits last 0.2 ms: the only way to reach the
    wait-ran-out path without breaking anything.  Used by tests/test_gpu_timeout.py;
    the product library never contains the injection."""
    build()
    out_dir = ROOT / "tests" / "_build"
    out_dir.mkdir(parents=True, exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    src, obj = CSRC / "plan_kernels.cu", OBJ / "plan_kernels.stall.o"
    if force or _stale(obj, [src, *headers]):
        _run([nvcc(), *NVCC_FLAGS, "-DRT_TEST_STALL", "-DRT_WAIT_NS=200000ull", "-c", str(src), "-o", str(obj)])
    names = CORE_CU + [f for f in OPTIONAL_CORE_CU if (CSRC / f).exists()] + \
        CORE_CPP + [f for f in OPTIONAL_CORE_CPP if (CSRC / f).exists()]
    objs = [obj if n == "plan_kernels.cu" else OBJ / (n + ".o") for n in names]
    lib = out_dir / "libretarget_b200_stall.so"
    if force or _stale(lib, objs):
        _run([nvcc(), "-shared", "-o", str(lib), *map(str, objs),
              "-cudart", "static", "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"])
    return lib


if __name__ == "__main__":
    built = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    for k, v in built.items():
        if k != "compiled":
            print(k, v)
