"""GPU parity of the tensor-pipe GEMV of wv_gemv_tc.cu (mma.sync m16n8k32 over tensor-map-fed tiles,
16-bit activation digits with a residual pass for vectors with outliers): every packed integer-code
format, shapes with one and several column segments, ragged last segments, row counts that are not
multiples of 16, against both restated references; inputs that must give exact zeros, that take the
residual pass, or that make rows non-finite."""
import numpy as np
import pytest

import oracle as O
from conftest import make_w, to_product_blob

pytestmark = pytest.mark.gpu
TOL = 1e-3
FORMATS = [("Q8_0", 0), ("Q4_0", 0), ("Q4_1", 0), ("Q5_0", 0), ("Q5_1", 0), ("Q2_K", 0), ("Q3_K", 0), ("Q4_K", 0), ("Q5_K", 0), ("Q6_K", 0),
           ("IQ1_S", 0), ("IQ2_XXS", 0), ("IQ2_XS", 0), ("IQ3_XXS", 0), ("IQ3_S", 0), ("IQ4_XS", 0), ("TernaryPacked", 0),
           ("BinaryPacked", 32), ("BinaryPacked", 128), ("AffinePacked", 64)]
SHAPES = [(100, 4096), (333, 14336), (48, 11264), (17, 1024), (2500, 2048)]


@pytest.fixture
def tc(wv, hooks):
    hooks.wv_set_tma_tuning(30, 0)
    yield wv
    hooks.wv_set_tma_tuning(0, 0)
    hooks.wv_set_act_width(0)


def _run(wv, f, bw, rows, cols, x, w=None):
    w = make_w(7, rows, cols)[0] if w is None else w
    ob = O.pack(f, w, rows, cols, bw)
    blob = to_product_blob(wv, ob)
    y = np.full(rows, np.nan, np.float32)
    wv.quant.MatVec(blob, x, y)
    assert wv._lib.lib().wv_device_status() == 0
    return y, ob


def _check(y, ob, x):
    den = O.sum_abs_wx(ob, x)
    for ref in (O.matvec(ob, x), O.matvec_simd(ob, x, 0)):
        err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
        assert np.all(err <= TOL * den + 1e-30), float(np.max(err / np.maximum(den, 1e-30)))


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda c: f"{c[0]}{c[1] or ''}")
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
def test_tc_matches_references(tc, fmt, shape):
    f, bw = fmt
    rows, cols = shape
    x = np.random.default_rng(11).normal(0, 1, cols).astype(np.float32)
    y, ob = _run(tc, f, bw, rows, cols, x)
    _check(y, ob, x)


@pytest.mark.parametrize("fmt", [("Q4_0", 0), ("Q4_K", 0), ("Q6_K", 0), ("IQ3_S", 0), ("BinaryPacked", 128), ("Q8_0", 0)], ids=lambda c: c[0])
def test_tc_residual_pass(tc, fmt):
    """Outliers inside 32-column blocks: the vector fails the 16-bit criterion and gets the residual pass; forcing
    that pass on an ordinary vector must not change the result beyond rounding."""
    f, bw = fmt
    rows, cols = 200, 4096
    x = np.random.default_rng(12).normal(0, 1, cols).astype(np.float32)
    xo = x.copy()
    xo[::97] *= 3000.0
    xo[64:96] = 0.0
    xo[128:160] *= 1e-30
    y, ob = _run(tc, f, bw, rows, cols, xo)
    _check(y, ob, xo)
    y1, _ = _run(tc, f, bw, rows, cols, x)
    tc._lib.lib().wv_set_act_width(3)
    y2, _ = _run(tc, f, bw, rows, cols, x)
    tc._lib.lib().wv_set_act_width(0)
    _check(y2, ob, x)
    den = O.sum_abs_wx(ob, x)
    assert np.all(np.abs(y1.astype(np.float64) - y2) <= 1e-4 * den + 1e-30)


@pytest.mark.parametrize("fmt", [("Q4_0", 0), ("Q8_0", 0), ("Q5_0", 0), ("Q6_K", 0), ("TernaryPacked", 0)], ids=lambda c: c[0])
def test_tc_zero_rows_are_exact(tc, fmt):
    f, bw = fmt
    rows, cols = 64, 4096
    w = make_w(3, rows, cols)[0]
    w[5] = 0.0
    w[40:48] = 0.0
    x = np.random.default_rng(5).normal(0, 3, cols).astype(np.float32)
    y, _ = _run(tc, f, bw, rows, cols, x, w)
    assert np.all(y[5] == 0.0) and np.all(y[40:48] == 0.0)
    assert np.all(np.isfinite(y))


def test_tc_nonfinite_and_zero_activations(tc):
    rows, cols = 32, 4096
    x = np.random.default_rng(6).normal(0, 1, cols).astype(np.float32)
    x[100] = np.inf
    y, _ = _run(tc, "Q4_0", 0, rows, cols, x)
    assert not np.any(np.isfinite(y))
    x = np.zeros(cols, np.float32)
    y, _ = _run(tc, "Q4_1", 0, rows, cols, x)
    assert np.all(y == 0.0)


def test_tc_batch_rows(tc):
    """batch > 1 through the host entry: every activation row gives its own output row."""
    rows, cols, batch = 96, 2048, 3
    w, _ = make_w(21, rows, cols)
    ob = O.pack("Q4_K", w, rows, cols)
    blob = to_product_blob(tc, ob)
    X = np.random.default_rng(22).normal(0, 1, (batch, cols)).astype(np.float32)
    Y = np.zeros((batch, rows), np.float32)
    key = tc.quant.EnsureResident(blob)
    tc._lib.check(tc._lib.lib().wv_matvec(key, X.ctypes.data, Y.ctypes.data, batch, cols, rows))
    for i in range(batch):
        _check(Y[i], ob, X[i])
