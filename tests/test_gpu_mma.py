"""GPU parity of the opt-in tensor-pipe GEMV (mma.sync m16n8k32 over tensor-map-fed tiles): the
formats it serves, at shapes with one and with several column segments, ragged last segments and
row counts that are not multiples of 16, against both restated references; plus inputs that
must give exact zeros or non-finite rows."""
import numpy as np
import pytest

import oracle as O
from conftest import make_w, to_product_blob

pytestmark = pytest.mark.gpu
TOL = 1e-3
FORMATS = [("Q8_0", 0), ("Q4_0", 0), ("Q4_1", 0), ("Q5_0", 0), ("Q5_1", 0), ("IQ1_S", 0), ("IQ2_XXS", 0), ("IQ3_XXS", 0),
           ("BinaryPacked", 32), ("BinaryPacked", 128), ("AffinePacked", 64)]
SHAPES = [(100, 4096), (4096, 4096), (333, 14336), (48, 11264), (17, 1024)]


@pytest.fixture
def mma(wv, hooks):
    hooks.wv_set_tma_tuning(24, 0)
    yield wv
    hooks.wv_set_tma_tuning(0, 0)


def _check(wv, f, bw, rows, cols, x, w=None):
    w = make_w(7, rows, cols)[0] if w is None else w
    ob = O.pack(f, w, rows, cols, bw)
    blob = to_product_blob(wv, ob)
    y = np.full(rows, np.nan, np.float32)
    wv.quant.MatVec(blob, x, y)
    return y, ob


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda c: f"{c[0]}{c[1] or ''}")
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
def test_mma_matches_references(mma, fmt, shape):
    f, bw = fmt
    rows, cols = shape
    if f == "BinaryPacked" and bw == 128 and cols % 128:
        pytest.skip("group 128 needs cols % 128 == 0")
    x = np.random.default_rng(11).normal(0, 1, cols).astype(np.float32)
    x[::97] *= 300.0   # outliers inside some 32-column blocks
    y, ob = _check(mma, f, bw, rows, cols, x)
    den = O.sum_abs_wx(ob, x)
    for ref in (O.matvec(ob, x), O.matvec_simd(ob, x, 0)):
        err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
        assert np.all(err <= TOL * den + 1e-30), float(np.max(err / np.maximum(den, 1e-30)))


@pytest.mark.parametrize("fmt", [("Q4_0", 0), ("Q8_0", 0), ("Q5_0", 0)], ids=lambda c: c[0])
def test_mma_zero_rows_are_exact(mma, fmt):
    f, bw = fmt
    rows, cols = 64, 4096
    w = make_w(3, rows, cols)[0]
    w[5] = 0.0
    w[40:48] = 0.0
    x = np.random.default_rng(5).normal(0, 3, cols).astype(np.float32)
    y, _ = _check(mma, f, bw, rows, cols, x, w)
    assert np.all(y[5] == 0.0) and np.all(y[40:48] == 0.0)
    assert np.all(np.isfinite(y))


def test_mma_nonfinite_activations(mma):
    rows, cols = 32, 4096
    x = np.random.default_rng(6).normal(0, 1, cols).astype(np.float32)
    x[100] = np.inf
    y, _ = _check(mma, "Q4_0", 0, rows, cols, x)
    assert not np.any(np.isfinite(y))
    x = np.zeros(cols, np.float32)
    y, _ = _check(mma, "Q4_1", 0, rows, cols, x)
    assert np.all(y == 0.0)
