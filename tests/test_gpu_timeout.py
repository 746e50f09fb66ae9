"""GPU: the bounded waits of the bulk-copy (TMA) staging kernel.

The product library cannot be made to miss a copy, so this test loads a TEST
BUILD of the same sources (retarget_b200.build.build_stall_variant: the
producer of CTA 0 skips its first copy; waits last 0.2 ms).  The consumers'
wait on that stage runs out, the launch drains, reports RT_RESULT_TIMEOUT and
commits nothing; the next launch on the same plan is unaffected.  Nothing in
here faults or hangs: an mbarrier that never completes is waited on for a
bounded time and then left alone."""
import json
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

SCRIPT = textwrap.dedent("""
    import json, sys, time
    import numpy as np
    sys.path.insert(0, %r)
    from oracle import compose
    from retarget_b200 import capi, workloads
    from retarget_b200.planner import DevicePlanner, ranges_to_tuples
    a = workloads.sparse_feedback(0, layers=4, requests=16)
    p = DevicePlanner(a.layout, 0, max_indices=a.n_idx + 8)
    before = [{1, 2}, set(), {5}, {7, 8, 9}]
    p.set_resident(before)
    out = {}
    t0 = time.perf_counter()
    try:
        p.step_host(a.slots, a.group_off, a.budget_blocks, capi.RT_PLAN_EVICT | capi.RT_PLAN_TMA)
        out["status"] = 0
    except capi.RtError as e:
        out["status"] = e.status
    out["seconds"] = time.perf_counter() - t0
    out["resident_kept"] = p.get_resident() == [sorted(s) for s in before]
    # the same plan handle, register-staged kernel: scratch was left clean
    resident = [set(s) for s in before]
    want, _ = compose.plan_step(a, resident, evict=True, literal=True)
    got, res = p.step_host(a.slots, a.group_off, a.budget_blocks, capi.RT_PLAN_EVICT)
    out["next_step_exact"] = ranges_to_tuples(got) == want and res.flags == 0
    out["next_resident_exact"] = p.get_resident() == [sorted(s) for s in resident]
    out["timeout_status"] = capi.RT_ERR_TIMEOUT
    p.close()
    print(json.dumps(out))
""") % str(ROOT)


def test_wait_that_runs_out_is_reported_and_commits_nothing():
    from retarget_b200 import build
    lib = build.build_stall_variant()
    env = dict(os.environ, RETARGET_B200_LIB=str(lib))
    proc = subprocess.run([sys.executable, "-c", SCRIPT], env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    out = json.loads(proc.stdout.strip().splitlines()[-1])
    assert out["status"] == out["timeout_status"]
    assert out["seconds"] < 2.0               # a handful of 0.2 ms waits, not one per work unit
    assert out["resident_kept"] and out["next_step_exact"] and out["next_resident_exact"]
