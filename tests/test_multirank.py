"""Two planner processes on CPU (gloo): rendezvous, barrier, max-over-ranks
and the all-ranks-agree check that the multi-GPU benchmark relies on.  Each rank
plans its own shard independently (here with the CPU oracle standing in for
the GPU) -- there is no data-path collective to test."""
import os
import socket
import subprocess
import sys
import textwrap
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

WORKER = textwrap.dedent("""
    import sys, json
    sys.path.insert(0, {root!r})
    from retarget_b200 import workloads
    from retarget_b200.multirank import Ranks
    from oracle import c_oracle
    r = Ranks({backend!r}).start()
    assert r.world == 2
    batch = workloads.tp_shard(0, requests=32)          # the same slot table on every rank
    co = c_oracle.COracle(batch.layout, device=r.local_rank)
    ranges, invalid = co.step(batch.slots, batch.group_off, batch.budget_blocks, True, 1)
    # dst is the rank's own GPU; everything else must agree
    plan = b"".join(ranges[k].tobytes() for k in ("buffer", "offset", "bytes"))
    r.barrier()
    same = r.same_everywhere(plan)
    differs = r.same_everywhere(bytes([r.rank]))
    mx = r.max_over_ranks([1.0 + r.rank, 5.0 - r.rank])
    if r.rank == 0:
        print(json.dumps(dict(same=same, differs=differs, mx=mx, n=len(ranges), dst=int(ranges["dst"][0]))))
    else:
        assert int(ranges["dst"][0]) == 1
    r.stop()
""")


import pytest


@pytest.mark.parametrize("backend", ["gloo", "file"])
def test_two_ranks_plan_independently_and_agree(tmp_path, backend):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=str(ROOT), backend=backend))
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2",
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (out, err) in zip(procs, outs):
        assert p.returncode == 0, err[-2000:]
    import json
    got = json.loads(outs[0][0].strip().splitlines()[-1])
    assert got["same"] is True and got["differs"] is False
    assert got["mx"] == [2.0, 5.0] and got["n"] > 0 and got["dst"] == 0
