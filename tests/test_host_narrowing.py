"""The host-side narrowing of slot ids (what the host-buffer planning call does
before the ids cross the host link): every id keeps its class -- below 1 stays
below 1, 1..2^31-1 is unchanged, anything larger ends above every capacity the
narrowed path accepts -- whatever the alignment, the length or the number of
threads."""
import ctypes as C

import numpy as np
import pytest

from retarget_b200 import capi


def narrow(src, threads, offset=0):
    buf = np.full(len(src) + offset + 8, 0x5a5a5a5a, dtype=np.int32)
    dst = buf[offset:offset + len(src)]
    fn = capi.lib.rt_narrow_ids
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32]
    assert fn(src.ctypes.data, dst.ctypes.data, len(src), threads) == 0
    # nothing outside the destination was written
    assert (buf[:offset] == 0x5a5a5a5a).all() and (buf[offset + len(src):] == 0x5a5a5a5a).all()
    return dst.copy()


def expected(src):
    out = np.where(src < 0, -1, np.minimum(src, 2**31 - 1))
    return out.astype(np.int32)


@pytest.mark.parametrize("threads", [1, 3, 8])
@pytest.mark.parametrize("n", [0, 1, 7, 8, 9, 65536, 65537, 300001])
def test_every_id_keeps_its_class(n, threads):
    rng = np.random.default_rng(n + threads)
    src = rng.integers(0, 262145, size=n + 3, dtype=np.int64)
    special = np.array([-1, 0, 1, 2**31 - 2, 2**31 - 1, 2**31, 2**32 - 1, 2**32, 2**40 + 5, -2**31, -2**31 - 1,
                        -2**40, np.iinfo(np.int64).min, np.iinfo(np.int64).max], dtype=np.int64)
    if n:
        at = rng.integers(0, len(src), size=min(len(special), n))
        src[at] = special[:len(at)]
    for src_off in (0, 1, 3):             # the source 8-, not 16- or 32-byte aligned
        for dst_off in (0, 1, 5):         # the destination off its 32-byte grid
            got = narrow(src[src_off:src_off + n], threads, dst_off)
            assert np.array_equal(got, expected(src[src_off:src_off + n]))


def test_default_thread_count_and_bad_arguments():
    src = np.arange(200000, dtype=np.int64)
    assert np.array_equal(narrow(src, 0), src.astype(np.int32))
    fn = capi.lib.rt_narrow_ids
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32]
    assert fn(None, None, 0, 1) == 0
    assert fn(None, None, 5, 1) == capi.RT_ERR_INVALID_ARGUMENT
