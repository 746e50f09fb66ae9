"""GPU parity over seeded random geometries: bitmap widths either side of every
word boundary, block sizes that are not powers of two, partial last blocks,
shared and per-layer bitmaps, budgets from one block to the whole buffer, ids
out of range mixed in.  Each case runs a few consecutive steps through the C ABI
and compares ranges, counters and the resident set with the CPU oracle, exactly."""
import dataclasses
import os
import math

import numpy as np
import pytest

from test_gpu_plan_parity import MODES, random_batch, run_steps

pytestmark = pytest.mark.gpu

# RETARGET_FUZZ_SEEDS=N runs a longer sweep of the same generator
SEEDS = int(os.environ.get("RETARGET_FUZZ_SEEDS", 24))

# bitmap widths worth hitting on purpose: around 32-bit words, around the widths
# the tail's segmented scans switch at, and the protocol's limit of 1024 blocks
EDGE_BLOCKS = [1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257, 511, 512, 513, 1000, 1023, 1024]


def random_shape(rng):
    bytes_per_slot = int(rng.choice([256, 512, 1024, 2048, 4096]))
    # a block is a whole number of slots and of 4 KiB pages
    unit = 4096 // math.gcd(4096, bytes_per_slot)
    block_tokens = unit * int(rng.integers(1, 7))
    n_blocks = int(rng.choice(EDGE_BLOCKS)) if rng.random() < .7 else int(rng.integers(1, 1025))
    # the last block is cut short in half of the cases
    # (a buffer smaller than one block is not a valid geometry)
    cut = int(rng.integers(0, block_tokens)) if n_blocks > 1 and rng.random() < .5 else 0
    pool_slots = max(2, n_blocks * block_tokens - cut)
    layers = int(rng.choice([1, 2, 3, 5, 8, 16]))
    n_req = int(rng.integers(1, 7))
    max_len = int(min(4000, max(8, pool_slots * rng.choice([.05, .5, 1.5]))))
    budget = int(rng.choice([1, max(1, n_blocks // 7), max(1, n_blocks // 2), n_blocks]))
    return dict(layers=layers, pool_slots=pool_slots, bytes_per_slot=bytes_per_slot,
                shared=bool(rng.random() < .4), n_req=n_req, max_len=max_len, budget=budget,
                block_bytes=block_tokens * bytes_per_slot)


@pytest.mark.parametrize("flags", MODES)
@pytest.mark.parametrize("seed", range(SEEDS))
def test_random_geometry(seed, flags):
    rng = np.random.default_rng(9000 + seed)
    shape = random_shape(rng)
    batches = [random_batch(rng, junk=(k == 1), **shape) for k in range(3)]
    # the budget shrinks on the last step, so blocks have to leave
    batches[2] = dataclasses.replace(batches[2], budget_blocks=max(1, shape["budget"] // 3))
    run_steps(batches, evict=bool(seed & 1), flags=flags)
