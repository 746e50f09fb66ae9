"""CPU-side checks of the C ABI: the library loads, exports everything the header
declares, and its host arithmetic equals the reference vectors and the oracle.
No device work is started here."""
import ctypes as C
import random
import re
from pathlib import Path

import numpy as np
import pytest

from oracle import ref_policy as rp
from oracle import uvm_expand as ux
from retarget_b200 import capi

ROOT = Path(__file__).resolve().parent.parent


def test_every_declared_symbol_is_exported():
    declared = set()
    for header in (ROOT / "include").glob("*.h"):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        declared |= set(re.findall(r"\b(rt_[a-z0-9_]+)\s*\(", text))
    assert len(declared) >= 20
    lib = C.CDLL(str(capi.LIB_PATH))
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, missing
    assert lib.rt_abi_version() == 1


def _spec(kw):
    full = dict(width_tokens=32768, lookahead_tokens=16384, quantum_tokens=8192)
    full.update(kw)
    return full


def test_window_matches_reference_vectors(golden):
    out = (C.c_uint64 * 2)()
    for name, block in golden["window"]["windows"].items():
        s = capi.window_spec_struct(**_spec(block["spec"]))
        assert capi.lib.rt_window_spec_check(C.byref(s), None) == 0, name
        for c, want in block["cases"]:
            assert capi.lib.rt_window(C.byref(s), float(c), out) == 0
            assert [out[0], out[1]] == want, (name, c)


def test_window_spec_messages(golden):
    for kw, message in golden["window"]["rejected"]:
        kw = _spec(kw)
        if type(kw.get("allocation_count")) is bool or kw.get("idle_only") == 1 and kw["idle_only"] is not True:
            continue   # Python-type checks have no C counterpart; the Python mirror covers them
        if "update_mode" in kw and kw["update_mode"] not in capi.UPDATE_MODES:
            continue
        s = capi.window_spec_struct(**kw)
        bad = C.c_int(-1)
        st = capi.lib.rt_window_spec_check(C.byref(s), C.byref(bad))
        assert st < 0
        text = capi.strerror(st)
        if st == capi.RT_ERR_SPEC_POSITIVE:
            names = ["allocation_bytes", "allocation_count", "bytes_per_token", "width_tokens",
                     "lookahead_tokens", "quantum_tokens"]
            assert message == f"cache_window.{names[bad.value]} must be a positive integer"
        else:
            assert text == message
    s = capi.window_spec_struct(448790528, 80, 2048, 32768, 16384, 8192)
    out = (C.c_uint64 * 2)()
    for bad_count in (-1.0, float("nan"), float("inf")):
        st = capi.lib.rt_window(C.byref(s), bad_count, out)
        assert capi.strerror(st) == "invalid completed-token count"


def test_interval_difference_and_accounting(golden):
    out = (C.c_uint64 * 4)()
    for a, b, want in golden["window"]["interval_difference"]:
        n = capi.lib.rt_interval_difference((C.c_uint64 * 2)(*a), (C.c_uint64 * 2)(*b), out)
        assert [[out[2 * i], out[2 * i + 1]] for i in range(n)] == want
    for mode, block in golden["window_controller"].items():
        s = capi.window_spec_struct(**block["spec"])
        allocs = block["allocations"]
        other = sum(a["bytes"] for a in allocs if a["bytes"] != block["spec"]["allocation_bytes"])
        n_cache = sum(1 for a in allocs if a["bytes"] == block["spec"]["allocation_bytes"])
        for step in block["log"]:
            res = step.get("result")
            if not res:
                continue
            old = res["old_window"] or [0, 0]
            g, c = C.c_uint64(), C.c_uint64()
            st = capi.lib.rt_window_accounting(
                C.byref(s), n_cache, other, (C.c_uint64 * 2)(*old),
                (C.c_uint64 * 2)(*res["new_window"]), int(res["initial"]),
                int(res["full_cache_refresh"]), C.byref(g), C.byref(c))
            assert st == 0
            assert (g.value, c.value) == (res["requested_gpu_bytes"], res["requested_cpu_bytes"])


def test_encode_mask_and_runs(golden):
    buf = C.create_string_buffer(300)
    for blocks, want in golden["runs"]["encode_mask"]:
        arr = (C.c_uint32 * max(1, len(blocks)))(*blocks)
        n = capi.lib.rt_encode_mask(arr, len(blocks), buf, 300)
        assert n == len(want) and buf.value.decode() == want
    for values, want in golden["runs"]["encode_runs"]:
        v = np.asarray(values, dtype=np.int64)
        runs = np.zeros((max(1, len(values)), 2), dtype=np.int64)
        n = C.c_size_t()
        st = capi.lib.rt_encode_runs(v.ctypes.data_as(C.POINTER(C.c_int64)), len(v),
                                     runs.ctypes.data_as(C.POINTER(C.c_int64)), len(runs), C.byref(n))
        assert st == 0 and runs[:n.value].tolist() == want


def test_slot_budget():
    s = capi.window_spec_struct(16 * 2097152, 4, 2048, 4096, 1024, 1024)
    b = C.c_uint64()
    assert capi.lib.rt_slot_budget(C.byref(s), 1024, C.byref(b)) == 0 and b.value == 4
    st = capi.lib.rt_slot_budget(C.byref(s), 3000, C.byref(b))
    assert capi.strerror(st) == "KV budget must be divisible by block_tokens"
    s2 = capi.window_spec_struct(16 * 2097152, 4, 3, 4096, 1024, 4096)
    st = capi.lib.rt_slot_budget(C.byref(s2), 1024, C.byref(b))
    assert capi.strerror(st) == "slot blocks must be page aligned"


# --------------------------------------------------------------------------
# plan-command expansion: C++ vs oracle restatement
# --------------------------------------------------------------------------
def _registry(rng, n_cache, alloc_bytes, extra):
    reg, nid = [], 1
    kinds = ["c"] * n_cache + ["x"] * extra
    rng.shuffle(kinds)
    for k in kinds:
        nid += rng.randint(1, 3)
        nbytes = alloc_bytes if k == "c" else rng.choice([4096, 12288, 1 << 20, 12345 * 4096, 4097])
        reg.append(dict(id=nid, bytes=nbytes, device=rng.choice([0, 0, 0, 3]),
                        concurrent=1 if rng.random() > 0.03 else 0))
    return reg


def _both(reg, gen, line):
    try:
        want = ux.command(reg, gen, line)
        want_err = None
    except ux.PlanError as e:
        want, want_err = None, str(e)
    got, got_err = capi.expand_command(reg, gen, line)
    assert got_err == want_err, (line, got_err, want_err)
    assert got == want, line


def test_expand_command_fuzz():
    rng = random.Random(1234)
    page = 4096
    for case in range(400):
        blk = rng.choice([page, 2 * page, 1 << 21, 512 * 1024])
        n_blocks = rng.choice([1, 2, 7, 64, 65, 1023, 1024])
        tail = rng.choice([0, 0, page, blk // 2]) if blk > page else 0
        alloc = blk * n_blocks - (tail if n_blocks > 1 else 0)
        reg = _registry(rng, rng.randint(1, 6), alloc, rng.randint(0, 3))
        n_cache = sum(1 for a in reg if a["bytes"] == alloc)
        gen = rng.randint(0, 5)
        # blocksv
        bits = [b for b in range(n_blocks) if rng.random() < rng.choice([0.05, 0.5, 0.95])]
        mask = rp.encode_mask(bits)
        use_gen = gen if rng.random() > .05 else gen + 1
        use_n = n_cache if rng.random() > .05 else n_cache + 1
        _both(reg, gen, f"blocksv {use_gen} {alloc} {use_n} {blk} {mask}")
        _both(reg, gen, f"blocksv {gen} {alloc} {n_cache} {blk} {mask}0")
        _both(reg, gen, f"blocksv {gen} {alloc} {n_cache} {blk + rng.choice([0, 1, page])} {mask}")
        # windows
        def edge():
            return min(alloc, rng.randint(0, n_blocks) * blk + rng.choice([0, 0, 0, 1, page]))
        o = sorted([edge(), edge()])
        w = sorted([edge(), edge()])
        if rng.random() < .2:
            o = [ux.UINT64_MAX, ux.UINT64_MAX]
        if rng.random() < .1:
            w[1] = alloc
        name = rng.choice(["windowv", "windowfullv"])
        _both(reg, gen, f"{name} {use_gen} {alloc} {use_n} {o[0]} {o[1]} {w[0]} {w[1]}")
        # prefix plans
        managed = sum(a["bytes"] for a in reg)
        t1 = rng.choice([0, managed, rng.randint(0, managed) // page * page, rng.randint(0, managed + 10)])
        t2 = rng.choice([0, managed, rng.randint(0, managed) // page * page])
        _both(reg, gen, f"target {t1}")
        _both(reg, gen, f"targetv {use_gen} {t1}")
        _both(reg, gen, f"retarget {use_gen} {t1} {t2}")
        a = rng.choice(reg)
        off = rng.choice([0, page, rng.randint(0, a["bytes"])])
        ln = rng.choice([page, a["bytes"] - min(off, a["bytes"]), rng.randint(0, a["bytes"])])
        _both(reg, gen, f"prefetch {a['id'] + rng.choice([0, 0, 0, 1000])} {off} {ln} {rng.choice(['cpu', 'gpu', 'tpu'])}")


@pytest.mark.parametrize("line", [
    "", "   ", "status extra", "windowv 1 2 3", "blocksv 0 4096 1 4096 1 extra1 extra2 extra3 extra4",
    "windowv 0 4096 1 0 0 0 x", "blocksv 0 4096 1 4096 G", "blocksv 0 4096 1 4096 F",
    "target 18446744073709551616", "target 18446744073709551615", "target -1", "target 1\t",
    "\ttarget\r 4096 ", "windowv\t0 4096 1 0 0 0 4096", "prefetch 1 0 4096 GPU",
    "blocksv 0 4096 1 4096 " + "1" * 257, "blocksv 0 4096 1 4096 " + "0" * 256,
])
def test_expand_command_odd_lines(line):
    reg = [dict(id=1, bytes=4096, device=0, concurrent=1)]
    _both(reg, 0, line)


# --------------------------------------------------------------------------
# host policy arithmetic on random inputs: C ABI vs the oracle (itself pinned
# to the reference's vectors above)
# --------------------------------------------------------------------------
def _random_window_spec(rng):
    """A spec that may or may not be valid: every rule of the reference's
    validation is broken some of the time."""
    bytes_per_token = rng.choice([256, 512, 1024, 2048, 4096, 3, 1536])
    quantum = rng.choice([16, 256, 1024, 8192, 24, 1000])
    width = quantum * rng.randint(1, 12) + (rng.choice([0, 0, 0, 1, quantum // 2]))
    lookahead = quantum * rng.randint(0, 12)
    allocation = width * bytes_per_token + rng.choice([-4096, 0, 0, 4096, 12345, 7 * quantum * bytes_per_token + 5])
    return dict(allocation_bytes=allocation, allocation_count=rng.randint(0, 80), bytes_per_token=bytes_per_token,
                width_tokens=width, lookahead_tokens=lookahead, quantum_tokens=quantum,
                min_update_seconds=rng.choice([0.0, 1.0, -1.0]))


def test_window_arithmetic_random_against_oracle():
    rng = random.Random(31)
    out = (C.c_uint64 * 2)()
    valid = 0
    for _ in range(3000):
        kw = _random_window_spec(rng)
        if any(kw[k] < 0 for k in ("allocation_bytes", "lookahead_tokens")):
            continue                                  # unsigned in the C structure
        spec = rp.WindowSpec(**kw)
        s = capi.window_spec_struct(**kw)
        st = capi.lib.rt_window_spec_check(C.byref(s), None)
        try:
            rp.check_window_spec(spec)
        except ValueError as e:
            message = str(e)
            if st == capi.RT_ERR_SPEC_POSITIVE:
                assert message.endswith("must be a positive integer"), kw
            else:
                assert capi.strerror(st) == message, kw
            continue
        assert st == 0, (kw, capi.strerror(st))
        valid += 1
        for _ in range(8):
            completed = rng.choice([0.0, rng.random() * 10, float(rng.randint(0, 1 << 22)),
                                    rng.random() * (1 << 22), float(1 << 53), 1e18, 3.5e300])
            assert capi.lib.rt_window(C.byref(s), completed, out) == 0
            assert (out[0], out[1]) == rp.window(spec, completed), (kw, completed)
    assert valid > 300


def test_interval_difference_random_against_oracle():
    rng = random.Random(32)
    out = (C.c_uint64 * 4)()
    for _ in range(5000):
        a = sorted(rng.randint(0, 40) for _ in range(2))
        b = sorted(rng.randint(0, 40) for _ in range(2))
        n = capi.lib.rt_interval_difference((C.c_uint64 * 2)(*a), (C.c_uint64 * 2)(*b), out)
        assert [(out[2 * i], out[2 * i + 1]) for i in range(n)] == rp.interval_difference(a, b), (a, b)


def test_runs_masks_and_budget_random_against_oracle():
    rng = random.Random(33)
    buf = C.create_string_buffer(300)
    for _ in range(500):
        blocks = [rng.randint(0, 1023) for _ in range(rng.randint(0, 60))]
        arr = (C.c_uint32 * max(1, len(blocks)))(*blocks)
        n = capi.lib.rt_encode_mask(arr, len(blocks), buf, 300)
        want = rp.encode_mask(blocks)
        assert n == len(want) and buf.value.decode() == want
        # consecutive stretches, repeats, steps back, negative ids
        values, v = [], rng.randint(-5, 50)
        for _ in range(rng.randint(0, 200)):
            v += rng.choice([1, 1, 1, 1, 0, 2, -1, rng.randint(-40, 40)])
            values.append(v)
        vals = np.asarray(values, dtype=np.int64)
        runs = np.zeros((max(1, len(values)), 2), dtype=np.int64)
        count = C.c_size_t()
        st = capi.lib.rt_encode_runs(vals.ctypes.data_as(C.POINTER(C.c_int64)), len(vals),
                                     runs.ctypes.data_as(C.POINTER(C.c_int64)), len(runs), C.byref(count))
        assert st == 0 and runs[:count.value].tolist() == rp.encode_runs(values)
    b = C.c_uint64()
    for _ in range(2000):
        width = rng.choice([256, 1024, 4096, 32768, 3000])
        bytes_per_token = rng.choice([3, 256, 2048, 4096, 1536])
        block_tokens = rng.choice([1, 2, 6, 16, 256, 1024, 3000, 65536])
        w = rp.WindowSpec(1 << 40, 4, bytes_per_token, width, 1, 1)
        s = capi.window_spec_struct(1 << 40, 4, bytes_per_token, width, 1, 1)
        st = capi.lib.rt_slot_budget(C.byref(s), block_tokens, C.byref(b))
        try:
            want = rp.slot_plan_budget(w, rp.SlotSpec(block_tokens=block_tokens))
        except ValueError as e:
            assert capi.strerror(st) == str(e), (width, bytes_per_token, block_tokens)
        else:
            assert st == 0 and b.value == want
