"""GPU parity of the event-driven path over seeded random geometries and
policies: block sizes that are not powers of two, bitmaps from two words to the
protocol's 1024 blocks, update limits from one block to the whole budget, active
and refresh periods shorter and longer than the trace, with and without
eviction, 64- and 32-bit ids, an allocator clear somewhere in the middle.  Every
step's range list, counters and resident set, and the snapshot every 16 steps,
must equal the CPU restatement of the reference's chain exactly.  Odd seeds drive
the device through the one-launch step, even seeds through the three calls."""
import os

import numpy as np
import pytest

from retarget_b200 import workloads
from test_gpu_feedback import run_trace

pytestmark = pytest.mark.gpu

# RETARGET_FUZZ_SEEDS=N runs a longer sweep of the same generator
SEEDS = int(os.environ.get("RETARGET_FUZZ_SEEDS", 16))


def random_case(rng):
    block_tokens = int(rng.choice([2, 6, 16, 24, 64, 256, 1024]))
    n_blocks = int(rng.choice([33, 64, 65, 200, 256, 257, 1000, 1024]))
    pool_slots = n_blocks * block_tokens - int(rng.integers(0, block_tokens))
    # the trace allocates whole 16-slot pages below the pool's end
    trace_slots = max(64, pool_slots // 16 * 16 - 16)
    budget = int(rng.choice([1, max(1, n_blocks // 8), max(1, n_blocks // 2), n_blocks]))
    return dict(
        layout=workloads.Layout(int(rng.choice([1, 2, 8])), 2048, pool_slots, block_tokens * 2048),
        trace=dict(steps=int(rng.integers(40, 90)), pool_slots=trace_slots,
                   arrival_rate=float(rng.choice([.3, 1.0, 2.5])),
                   median=int(min(max(8, trace_slots // 40), 512)), mean_output=int(rng.choice([4, 24, 80])),
                   initial_requests=int(rng.integers(0, 8))),
        policy=dict(budget=budget, max_blocks=int(rng.choice([1, 4, max(1, budget // 2), budget])),
                    active=float(rng.choice([.05, .5, 5.0])), refresh=float(rng.choice([.1, 1.0, 20.0])),
                    evict=bool(rng.random() < .6)),
        clear_at=int(rng.integers(10, 35)) if rng.random() < .4 else None,
        dtype=np.int32 if rng.random() < .5 else np.int64)


@pytest.mark.parametrize("seed", range(SEEDS))
def test_random_policy_and_geometry(seed):
    rng = np.random.default_rng(7100 + seed)
    case = random_case(rng)
    trace = workloads.decode_trace(int(rng.integers(1 << 30)), **case["trace"])
    run_trace(case["layout"], trace, clear_at=case["clear_at"], dtype=case["dtype"], fused=bool(seed & 1),
              **case["policy"])
