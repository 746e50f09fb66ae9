"""The read-only bandwidth yardstick reads every byte it is given: its sink is
the xor of all 64-bit words, folded the way the kernel folds them."""
import ctypes as C

import numpy as np
import pytest

from retarget_b200 import capi

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.mark.parametrize("n_words", [2, 2046, 2048, 2050, 1 << 20, (1 << 22) + 6])
def test_sink_is_the_fold_of_every_word(n_words):
    rng = np.random.default_rng(n_words)
    data = rng.integers(0, 1 << 63, size=n_words, dtype=np.int64).view(np.uint32).reshape(-1, 4)
    # per 16-byte vector (x, y, z, w): high half x ^ z, low half y ^ w
    hi = np.bitwise_xor.reduce(data[:, 0] ^ data[:, 2]).astype(np.uint64)
    lo = np.bitwise_xor.reduce(data[:, 1] ^ data[:, 3]).astype(np.uint64)
    want = int((hi << np.uint64(32)) | lo)
    dev = torch.device("cuda:0")
    d = torch.from_numpy(data.view(np.int64).reshape(-1).copy()).to(dev)
    sink = torch.zeros(1, dtype=torch.int64, device=dev)
    fn = capi.lib.rt_read_probe
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]
    capi.check(fn(d.data_ptr(), 8 * n_words, sink.data_ptr(), None), "rt_read_probe")
    torch.cuda.synchronize()
    assert int(sink.cpu().numpy().view(np.uint64)[0]) == want
    assert fn(d.data_ptr() + 8, 16, sink.data_ptr(), None) == capi.RT_ERR_INVALID_ARGUMENT
