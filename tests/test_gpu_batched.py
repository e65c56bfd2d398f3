"""Batched Dense MatVec (several activation rows against one packed matrix) on the tcgen05 kernel: every packed
format, batches around the padding and tiling edges, rows that do not fill the last 128-row tile, against the oracle's
SIMD-path GEMV per activation row within 1e-3 * sum |w x|, and the small-batch GEMM configuration at full size."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O
from conftest import CASES, case_id, case_ok, to_product_blob

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _run(wv, ob, x):
    """x: [batch, cols] -> y [batch, rows] through wv_matvec_dev with device buffers."""
    L = wv._lib.lib()
    blob = to_product_blob(wv, ob)
    key = wv.quant.EnsureResident(blob)
    dx = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    dy = torch.full((x.shape[0], ob.rows), float("nan"), device="cuda")
    wv._lib.check(L.wv_matvec_dev(key, dx.data_ptr(), dy.data_ptr(), x.shape[0], ob.cols, ob.rows, None))
    torch.cuda.synchronize()
    assert L.wv_device_status() == 0
    return dy.cpu().numpy(), blob


def _check(ob, x, y, rows_checked=None):
    cache = O.SimdCache(ob)
    worst = 0.0
    for m in (range(x.shape[0]) if rows_checked is None else rows_checked):
        ref = np.zeros(ob.rows, np.float32)
        cache.matvec(np.ascontiguousarray(x[m]), ref, 0)
        den = O.sum_abs_wx(ob, x[m])
        err = np.abs(y[m].astype(np.float64) - ref)
        assert np.all(err <= TOL * den + 1e-30), (m, float(np.max(err / np.maximum(den, 1e-30))))
        worst = max(worst, float(np.max(err / np.maximum(den, 1e-30))))
    return worst


@pytest.mark.parametrize("case", [c for c in CASES if c[0] != "none"], ids=case_id)
@pytest.mark.parametrize("batch", [2, 16, 17, 100])
def test_batched_every_format(wv, case, batch):
    f, bw, dt = case
    rows, cols = 300, 1024            # three row tiles, the last one 44 rows; four column splits
    w = np.random.default_rng(21).normal(0, 0.02, rows * cols).astype(np.float32)
    ob = O.pack(f, w, rows, cols, bw, dt)
    x = np.random.default_rng(22).normal(0, 1, (batch, cols)).astype(np.float32)
    x[0, ::5] *= 50.0                 # a row with outliers, and one scaled far down
    x[-1] *= 1e-20
    y, _ = _run(wv, ob, x)
    assert np.all(np.isfinite(y))
    _check(ob, x, y)


@pytest.mark.parametrize("fmt", ["Q8_0", "Q4_K"])
@pytest.mark.parametrize("batch", [1, 4, 16, 64, 256, 300])
def test_small_batch_gemm_configuration(wv, fmt, batch):
    """M activation rows x 4096 against W 4096 x 4096 in Q8_0 and in the 4-bit k-quant, N(0, 0.02^2) seed 3."""
    rows = cols = 4096
    rng = np.random.default_rng(3)
    w = rng.normal(0, 0.02, rows * cols).astype(np.float32)
    x = rng.normal(0, 1, (batch, cols)).astype(np.float32)
    ob = O.pack(fmt, w, rows, cols)
    y, blob = _run(wv, ob, x)
    picks = sorted({0, batch // 2, batch - 1})
    worst = _check(ob, x, y, picks)
    assert worst < TOL
    if batch > 1:
        # every row agrees with the batch-1 kernel's result for that row within the two kernels' error budgets
        L = wv._lib.lib()
        key = wv.quant.EnsureResident(blob)
        dx = torch.from_numpy(x).cuda()
        one = torch.zeros(rows, device="cuda")
        for m in picks:
            wv._lib.check(L.wv_matvec_dev(key, dx.data_ptr() + 4 * m * cols, one.data_ptr(), 1, cols, rows, None))
            torch.cuda.synchronize()
            den = O.sum_abs_wx(ob, x[m])
            assert np.all(np.abs(y[m].astype(np.float64) - one.cpu().numpy()) <= 2 * TOL * den + 1e-30)


def test_batched_wide_and_tall_shapes(wv):
    for rows, cols, batch in ((14336, 4096, 8), (4096, 14336, 33), (128, 32768, 5), (1000, 256, 256)):
        w = np.random.default_rng(rows).normal(0, 0.02, rows * cols).astype(np.float32)
        ob = O.pack("Q4_K", w, rows, cols)
        x = np.random.default_rng(cols).normal(0, 1, (batch, cols)).astype(np.float32)
        y, _ = _run(wv, ob, x)
        _check(ob, x, y, [0, batch - 1])


def test_dense_forward_batched(wv):
    """dense.Forward with a batch: bias and activation after the batched GEMV, as for batch 1."""
    d = wv.dense
    rows, cols, batch = 512, 2048, 24
    w = np.random.default_rng(5).normal(0, 0.02, rows * cols).astype(np.float32)
    layer = d.NewConfigured(cols, rows, d.ActivationSilu, wv.quant.DTypeFloat32, wv.quant.Format.FormatQ4_K, w)
    st = layer.Weights
    st.Bias = np.random.default_rng(6).normal(0, 0.1, rows)
    x = np.random.default_rng(7).normal(0, 1, (batch, cols)).astype(np.float32)
    pre, post = d.Forward(layer, x)
    ob = O.Blob(O.FMT["Q4_K"], rows, cols, st.Packed.Raw, st.Packed.Scales, st.Packed.Mins, st.Packed.BlockWeights)
    for m in (0, batch - 1):
        ref = O.matvec_simd(ob, x[m]).astype(np.float64) + st.Bias
        den = O.sum_abs_wx(ob, x[m])
        assert np.all(np.abs(pre[m] - ref) <= TOL * den + 1e-6)
        pm = pre[m].astype(np.float64)
        assert np.allclose(post[m], pm / (1 + np.exp(-pm)), rtol=1e-5, atol=1e-6)


def test_host_pointer_calls_from_threads(wv):
    """wv_matvec (host pointers in and out) from six threads at once, as goroutines call Dense in the reference: the
    staging slots keep the calls apart, every result equals the single-threaded one bit for bit."""
    import threading
    q = wv.quant
    rng = np.random.default_rng(31)
    jobs = []
    for i, (fmt, rows, cols) in enumerate((("Q4_K", 512, 4096), ("Q8_0", 300, 2048), ("IQ3_S", 1000, 1024), ("Q4_0", 96, 14336),
                                           ("Q6_K", 700, 2048), ("BinaryPacked", 256, 4096))):
        w = rng.normal(0, 0.02, rows * cols).astype(np.float32)
        blob = q.Pack(q.Format["Format" + fmt], w, rows, cols)
        x = rng.normal(0, 1, cols).astype(np.float32)
        want = np.zeros(rows, np.float32)
        q.MatVec(blob, x, want)
        jobs.append((blob, x, want))
    errors = []

    def worker(job):
        blob, x, want = job
        try:
            for _ in range(50):
                y = np.full(blob.Rows, np.nan, np.float32)
                q.MatVec(blob, x, y)
                if not np.array_equal(y.view(np.uint32), want.view(np.uint32)):
                    errors.append("mismatch")
                    return
        except Exception as e:   # noqa: BLE001
            errors.append(repr(e))
    threads = [threading.Thread(target=worker, args=(j,)) for j in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:3]
    assert wv._lib.lib().wv_device_status() == 0
