"""Greedy pick on the device against the restated sampling.ArgMax: ties keep the first index, NaN
never wins, NaN in position 0 keeps index 0, sizes around the thread count and the LM-head size."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 2, 31, 1024, 1025, 4097, 128256])
def test_argmax_matches_reference(wv, n):
    rng = np.random.default_rng(n)
    cases = [rng.normal(0, 3, n).astype(np.float32)]
    t = rng.integers(-3, 4, n).astype(np.float32)            # many ties
    cases.append(t)
    c = rng.normal(0, 1, n).astype(np.float32); c[n // 2] = np.nan; cases.append(c)   # NaN in the middle never wins
    c = rng.normal(0, 1, n).astype(np.float32); c[0] = np.nan; cases.append(c)        # NaN first: index 0
    cases.append(np.full(n, -np.inf, np.float32))
    c = np.zeros(n, np.float32); c[-1] = np.inf; cases.append(c)
    for v in cases:
        d = torch.from_numpy(v).cuda()
        assert wv.sampling.ArgMaxCUDA(d.data_ptr(), n) == O.argmax(v)


def test_argmax_after_lm_head_gemv(wv):
    rows, cols = 32000, 2048
    w = np.random.default_rng(1).normal(0, 0.02, rows * cols).astype(np.float32)
    blob = wv.quant.Pack(wv.quant.Format.FormatQ8_0, w, rows, cols)
    x = np.random.default_rng(2).normal(0, 1, cols).astype(np.float32)
    key = wv.quant.EnsureResident(blob)
    dx = torch.from_numpy(x).cuda()
    dy = torch.zeros(rows, device="cuda")
    L = wv._lib.lib()
    wv._lib.check(L.wv_matvec_dev(key, dx.data_ptr(), dy.data_ptr(), 1, cols, rows, None))
    got = wv.sampling.ArgMaxCUDA(dy.data_ptr(), rows)
    assert got == O.argmax(dy.cpu().numpy())
