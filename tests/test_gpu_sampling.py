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


@pytest.mark.parametrize("n,k", [(5, 3), (40, 40), (1000, 1), (1000, 0), (4097, 40), (32000, 50), (128256, 40), (128256, 1024), (128256, 7)])
def test_topk_sample_matches_reference(wv, n, k):
    """sampling.SampleTopK on the device against its restatement: the same candidate set, order and float64 walk,
    for draws across [0, 1] (the ends included), with many equal logits, and for the greedy short-cuts."""
    rng = np.random.default_rng(n * 31 + k)
    cases = [rng.normal(0, 3, n).astype(np.float32), rng.integers(-3, 4, n).astype(np.float32)]
    c = rng.normal(0, 1, n).astype(np.float32); c[::7] = c[3]; cases.append(c)           # equal values around the cut
    c = rng.normal(0, 1, n).astype(np.float32); c[n // 3] = -np.inf; c[n // 2] = 40.0; cases.append(c)
    draws = [0.0, 1e-12, 0.03, 0.25, 0.5, 0.77, 0.999999, 1.0]
    for v in cases:
        d = torch.from_numpy(v).cuda()
        for temp in (1.0, 0.7, 2.5):
            for u in draws:
                got = wv.sampling.SampleTopKCUDA(d.data_ptr(), n, k, temp, False, u)
                assert got == O.topk_sample(v, k, temp, False, u), (n, k, temp, u)
        assert wv.sampling.SampleTopKCUDA(d.data_ptr(), n, k, 0.0, False, 0.3) == O.argmax(v)     # temperature <= 0
        assert wv.sampling.SampleTopKCUDA(d.data_ptr(), n, k, 1.0, True, 0.3) == O.argmax(v)      # deterministic
        assert wv.sampling.SampleTopKCUDA(d.data_ptr(), n, 1, 1.0, False, 0.3) == O.argmax(v)     # topK == 1


def test_topk_sample_limits_and_distribution(wv):
    v = np.random.default_rng(9).normal(0, 2, 5000).astype(np.float32)
    d = torch.from_numpy(v).cuda()
    with pytest.raises(wv.WelvetError):       # every logit of 5000 is more than the device sampler takes
        wv.sampling.SampleTopKCUDA(d.data_ptr(), 5000, 0, 1.0, False, 0.5)
    with pytest.raises(wv.WelvetError):
        wv.sampling.SampleTopKCUDA(d.data_ptr(), 5000, 40, 1.0, False, 1.5)
    # frequencies over a grid of draws follow the softmax of the top 8
    k, temp = 8, 1.3
    top = np.argsort(-v, kind="stable")[:k]
    p = np.exp((v[top] / np.float32(temp) - v[top[0]] / np.float32(temp)).astype(np.float64)); p /= p.sum()
    us = (np.arange(2000) + 0.5) / 2000
    picks = np.array([wv.sampling.SampleTopKCUDA(d.data_ptr(), 5000, k, temp, False, float(u)) for u in us])
    assert set(picks) <= set(top.tolist())
    freq = np.array([(picks == t).mean() for t in top])
    assert np.abs(freq - p).max() < 2e-3
