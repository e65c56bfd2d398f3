"""Projection groups in one launch (`wv_matvec_dev_multi`): Q|K|V and gate|up shapes. The grouped
launch must give bit for bit what the separate launches of the same kernel give, and both must be
within the reference bound; mixed groups fall back to separate launches."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O
from conftest import make_w, to_product_blob

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _stores(wv, f, shapes, cols, seed):
    obs, sts = [], []
    for i, rows in enumerate(shapes):
        w, _ = make_w(seed + i, rows, cols)
        ob = O.pack(f, w, rows, cols)
        obs.append(ob)
        sts.append(wv.weights.FromBlob(to_product_blob(wv, ob)))
    return obs, sts


@pytest.mark.parametrize("fmt", ["Q4_K", "Q8_0", "Q4_0", "IQ3_S"])
@pytest.mark.parametrize("shapes", [(4096, 1024, 1024), (1500, 1500), (96, 40, 8, 300)], ids=["qkv", "gate_up", "four_ragged_rows"])
@pytest.mark.parametrize("batch", [1, 3])
def test_group_equals_separate_launches(wv, hooks, fmt, shapes, batch):
    cols = 4096
    L = wv._lib.lib()
    obs, sts = _stores(wv, fmt, shapes, cols, 40)
    x = np.random.default_rng(9).normal(0, 1, (batch, cols)).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    ys = [torch.full((batch, r), float("nan"), device="cuda") for r in shapes]
    wv.dense.MatVecGroupCUDA(sts, dx.data_ptr(), [y.data_ptr() for y in ys], batch, cols)
    torch.cuda.synchronize()
    assert L.wv_device_status() == 0
    L.wv_set_tma_tuning(14, 0)       # the separate launches on the same (dp4a) kernel
    try:
        for ob, st, y in zip(obs, sts, ys):
            ref = torch.zeros_like(y)
            key = wv.quant.EnsureResident(st.Packed)
            wv._lib.check(L.wv_matvec_dev(key, dx.data_ptr(), ref.data_ptr(), batch, cols, ob.rows, None))
            torch.cuda.synchronize()
            assert torch.equal(y.view(torch.int32), ref.view(torch.int32))
            got = y.cpu().numpy()
            for b in (0, batch - 1):
                den = O.sum_abs_wx(ob, x[b])
                want = O.matvec_simd(ob, x[b], 0)
                assert np.all(np.abs(got[b].astype(np.float64) - want) <= TOL * den + 1e-30)
    finally:
        L.wv_set_tma_tuning(0, 0)


def test_mixed_group_runs_as_separate_launches(wv):
    cols = 2048
    obs_a, st_a = _stores(wv, "Q4_K", (256,), cols, 60)
    obs_b, st_b = _stores(wv, "Q8_0", (128,), cols, 61)
    x = np.random.default_rng(3).normal(0, 1, cols).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    ys = [torch.zeros(256, device="cuda"), torch.zeros(128, device="cuda")]
    wv.dense.MatVecGroupCUDA(st_a + st_b, dx.data_ptr(), [y.data_ptr() for y in ys], 1, cols)
    torch.cuda.synchronize()
    for ob, y in zip(obs_a + obs_b, ys):
        den = O.sum_abs_wx(ob, x)
        assert np.all(np.abs(y.cpu().numpy().astype(np.float64) - O.matvec_simd(ob, x, 0)) <= TOL * den + 1e-30)


def test_group_argument_errors(wv):
    L = wv._lib.lib()
    keys = (C.c_uint64 * 5)(1, 2, 3, 4, 5)
    outs = (C.c_int * 5)(1, 1, 1, 1, 1)
    dys = (C.c_void_p * 5)(8, 8, 8, 8, 8)
    dx = torch.zeros(32, device="cuda")
    assert L.wv_matvec_dev_multi(keys, 5, dx.data_ptr(), dys, 1, 32, outs, None) == wv._lib.WV_EARG
    assert L.wv_matvec_dev_multi(keys, 2, dx.data_ptr(), dys, 1, 32, outs, None) == wv._lib.WV_ENOTFOUND
