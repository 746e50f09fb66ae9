"""The LD_PRELOAD library under the real driver: a PyTorch process started with
it gets its device allocations converted to registered managed allocations
(select.cpp:24724-24761), answers the control socket, and keeps computing
correct results while a controller outside moves its memory to the CPU and back."""
import os
import subprocess
import sys
import time
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

ROOT = Path(__file__).resolve().parent.parent
PRELOAD = ROOT / "retarget_b200" / "libretarget_preload.so"

CHILD = r"""
import os, sys, torch
a = torch.full((64 << 20,), 3, dtype=torch.uint8, device="cuda")          # 64 MiB
b = torch.arange(16 << 20, device="cuda", dtype=torch.int32)               # 64 MiB
c = (b[: 1 << 20].to(torch.float32) * 2).sum()
torch.cuda.synchronize()
print("READY", os.getpid(), flush=True)
for line in sys.stdin:                      # one round of work per line from the parent
    if line.strip() == "quit":
        break
    total = int(a.to(torch.int64).sum().item())
    last = int(b[-1].item())
    b += 1
    torch.cuda.synchronize()
    print("WORK", total, last, float(c.item()), flush=True)
"""


def test_pytorch_process_under_the_preload_library():
    from retarget_b200.control import UvmController
    env = dict(os.environ, LD_PRELOAD=str(PRELOAD), SELECT_UVM_ENABLE="1", SELECT_UVM_CONVERT_ALLOC="1",
               SELECT_UVM_CHUNK_MB="16", PYTORCH_NO_CUDA_MEMORY_CACHING="0")
    env.pop("RETARGET_B200_LIBCUDA", None)
    child = subprocess.Popen([sys.executable, "-c", CHILD], env=env, stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                             stderr=subprocess.PIPE, text=True)
    try:
        line = child.stdout.readline()
        assert line.startswith("READY"), (line, child.stderr.read() if child.poll() is not None else "")
        pid = int(line.split()[1])
        uvm = UvmController(pid)
        st = uvm.status()
        assert st.pid == pid and st.allocation_count >= 2 and st.managed_bytes >= 128 << 20
        assert os.path.exists(uvm.path) and (os.stat(uvm.path).st_mode & 0o777) == 0o600

        def work():
            child.stdin.write("go\n")
            child.stdin.flush()
            parts = child.stdout.readline().split()
            assert parts and parts[0] == "WORK", (parts, child.stderr.read() if child.poll() is not None else "")
            return int(parts[1]), int(parts[2]), float(parts[3])

        expect_last = (16 << 20) - 1
        assert work() == (3 * (64 << 20), expect_last, float(((1 << 20) - 1) * (1 << 20)))
        # everything the process owns goes to the CPU; it keeps working (pages fault back in)
        res = uvm.set_target(0, timeout=120)
        assert res.submitted_bytes == 0
        after = uvm.status()
        assert after.last_error == 0 and after.completed_cpu_bytes >= st.managed_bytes
        assert work()[:2] == (3 * (64 << 20), expect_last + 1)
        # and back, incrementally in two steps
        half = uvm.retarget(0, st.managed_bytes // 2, timeout=120)
        full = uvm.retarget(st.managed_bytes // 2, 1 << 50, timeout=120)
        assert half.submitted_bytes <= st.managed_bytes // 2 < full.submitted_bytes
        assert uvm.status().last_error == 0
        assert work()[:2] == (3 * (64 << 20), expect_last + 2)
        child.stdin.write("quit\n")
        child.stdin.flush()
        assert child.wait(timeout=60) == 0, child.stderr.read()
        deadline = time.time() + 5
        while os.path.exists(uvm.path) and time.time() < deadline:
            time.sleep(0.05)
        assert not os.path.exists(uvm.path)          # the library removes the socket it created
    finally:
        if child.poll() is None:
            child.kill()
