"""GPU: the synthetic paged decode-attention reader against a NumPy fp32
reference of the same arithmetic (bf16 inputs, fp32 accumulation; tolerance
1e-2 relative, the precision of one bf16 rounding of the inputs' products)."""
import ctypes as C

import numpy as np
import pytest

from retarget_b200 import capi

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def bind():
    fn = capi.lib.rt_paged_attention
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                   C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p]
    return fn


@pytest.mark.parametrize("heads", [8, 1, 3])
def test_paged_attention_matches_numpy(heads):
    fn = bind()
    rng = np.random.default_rng(4)
    dev = torch.device("cuda:0")
    layers, pool, dim = 3, 4096, 128
    K = [torch.randn(pool, heads, dim, device=dev).to(torch.bfloat16) for _ in range(layers)]
    V = [torch.randn(pool, heads, dim, device=dev).to(torch.bfloat16) for _ in range(layers)]
    lens = [1, 7, 300, 0, 1025, 64]
    slots = [rng.integers(1, pool, n) for n in lens]
    slots[2][::17] = 0                         # the padding slot is skipped
    slots[4][5] = slots[4][6]                  # a repeated slot counts twice
    slots[5][3] = pool + 77                    # outside the pool: skipped
    flat = np.concatenate(slots).astype(np.int64)
    off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    R = len(lens)
    q = torch.randn(R, layers, heads, dim, device=dev).to(torch.bfloat16)
    out = torch.full((R, layers, heads, dim), float("nan"), dtype=torch.float32, device=dev)
    kp = torch.tensor([t.data_ptr() for t in K], dtype=torch.int64, device=dev)
    vp = torch.tensor([t.data_ptr() for t in V], dtype=torch.int64, device=dev)
    d_slots, d_off = torch.from_numpy(flat).to(dev), torch.from_numpy(off).to(dev)
    torch.cuda.synchronize()
    st = fn(kp.data_ptr(), vp.data_ptr(), layers, heads, q.data_ptr(), d_slots.data_ptr(), d_off.data_ptr(), R,
            pool - 1, out.data_ptr(), None)
    assert st == 0, capi.strerror(st)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    qf = q.float().cpu().numpy()
    for r in range(R):
        ids = slots[r][(slots[r] >= 1) & (slots[r] <= pool - 1)]
        for l in range(layers):
            k = K[l].float().cpu().numpy()[ids]          # [n, heads, dim]
            v = V[l].float().cpu().numpy()[ids]
            for h in range(heads):
                if len(ids) == 0:
                    assert np.all(got[r, l, h] == 0)
                    continue
                s = (k[:, h] @ qf[r, l, h]) / np.sqrt(dim)
                p = np.exp(s - s.max())
                want = (p / p.sum()) @ v[:, h]
                np.testing.assert_allclose(got[r, l, h], want, rtol=1e-2, atol=1e-3)
