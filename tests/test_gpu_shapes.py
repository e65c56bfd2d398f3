"""GPU parity at the benchmark's shapes and on the kernel-selection boundaries: golden
fixtures, the 4096x4096 single-MatVec config, Llama FFN shapes, columns that take the
register-load kernel instead of the TMA-fed one, activations with outliers / zeros / inf,
and size-independent properties (linearity, row-shard reassembly) at full size."""
import os

import numpy as np
import pytest

import oracle as O
from conftest import CASES, case_id, case_ok, make_w, to_product_blob

pytestmark = pytest.mark.gpu
TOL = 1e-3
GOLD = os.path.join(os.path.dirname(__file__), "golden", "golden_small.npz")


def check(y, ob, x, refs=("scalar", "simd")):
    den = O.sum_abs_wx(ob, x)
    for name in refs:
        ref = O.matvec(ob, x) if name == "scalar" else O.matvec_simd(ob, x, 0)
        err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
        assert np.all(err <= TOL * den + 1e-30), f"{name}: worst {np.max(err / np.maximum(den, 1e-30)):.3e}"
    return float(np.max(np.abs(y.astype(np.float64) - O.matvec_simd(ob, x, 0)) / np.maximum(den, 1e-30)))


def test_golden_fixtures_on_device(wv):
    g = np.load(GOLD)
    q = wv.quant
    for rows, cols in ((8, 512), (3, 100)):
        x = g[f"x_{rows}x{cols}"]
        for c in CASES:
            if not case_ok(c, rows, cols):
                continue
            f, bw, dt = c
            k = f"{case_id(c)}_{rows}x{cols}"
            blob = q.Blob(q.Format(O.FMT[f]), rows, cols, g[k + "_raw"], g[k + "_scales"], g[k + "_mins"], bw or 0, dt)
            assert np.array_equal(q.Unpack(blob).view(np.uint32), g[k + "_unpack"].view(np.uint32)), k
            y = np.zeros(rows, np.float32)
            q.MatVec(blob, x, y)
            ob = O.Blob(O.FMT[f], rows, cols, g[k + "_raw"], g[k + "_scales"], g[k + "_mins"], blob.BlockWeights if f != "none" else 1, dt)
            if f == "BinaryPacked":
                ob.block_weights = 128 if bw == 128 else 32
            den = O.sum_abs_wx(ob, x)
            assert np.all(np.abs(y.astype(np.float64) - g[k + "_y_scalar"]) <= TOL * den + 1e-30), k


@pytest.mark.parametrize("case", CASES, ids=case_id)
def test_single_matvec_4096x4096(wv, case):
    """The single Dense MatVec config (4096x4096, W ~ N(0,0.02^2) seed 0, x ~ N(0,1) seed 1) for every layout."""
    f, bw, dt = case
    rows = cols = 4096
    w = np.random.default_rng(0).normal(0, 0.02, (rows, cols)).astype(np.float32)
    x = np.random.default_rng(1).normal(0, 1, cols).astype(np.float32)
    q = wv.quant
    blob = q.Pack(q.Format(O.FMT[f]), w, rows, cols, bw, dt)          # device packer
    ob = O.Blob(O.FMT[f], rows, cols, blob.Raw, blob.Scales, blob.Mins, blob.BlockWeights, dt)
    assert np.array_equal(q.Unpack(blob).view(np.uint32), O.unpack(ob).view(np.uint32))
    y = np.zeros(rows, np.float32)
    wv.dense.MatVecPackedBlob(blob, x, y)
    check(y, ob, x)


@pytest.mark.parametrize("fmt", ["Q4_K", "Q8_0", "Q4_0", "IQ2_XS", "IQ4_NL", "BinaryPacked"])
@pytest.mark.parametrize("shape", [(4096, 14336), (14336, 4096)], ids=["4096x14336", "14336x4096"])
def test_ffn_shapes_full_size(wv, fmt, shape):
    rows, cols = shape
    bw = 128 if fmt == "BinaryPacked" else 0
    w = np.random.default_rng(2).normal(0, 0.02, rows * cols).astype(np.float32)
    x = np.random.default_rng(22).normal(0, 1, cols).astype(np.float32)
    q = wv.quant
    blob = q.Pack(q.Format(O.FMT[fmt]), w, rows, cols, bw)
    ob = O.Blob(O.FMT[fmt], rows, cols, blob.Raw, blob.Scales, blob.Mins, blob.BlockWeights)
    assert np.array_equal(blob.Raw, O.pack(fmt, w, rows, cols, bw).raw), "device packer differs from the reference packer at full size"
    y = np.zeros(rows, np.float32)
    q.MatVec(blob, x, y)
    check(y, ob, x, refs=("simd",))
    # linearity: W(2x + x2) == 2 Wx + W x2 within tolerance (no oracle involved)
    x2 = np.random.default_rng(23).normal(0, 1, cols).astype(np.float32)
    y2, y3 = np.zeros(rows, np.float32), np.zeros(rows, np.float32)
    q.MatVec(blob, x2, y2)
    q.MatVec(blob, (2 * x + x2).astype(np.float32), y3)
    den = O.sum_abs_wx(ob, np.abs(2 * x) + np.abs(x2))
    assert np.all(np.abs(y3.astype(np.float64) - (2.0 * y + y2)) <= 3 * TOL * den)


_FULL = ("Q4_K", "Q8_0", "Q4_0", "IQ2_XS", "IQ4_NL", "BinaryPacked")   # covered by test_ffn_shapes_full_size (packer equality, linearity)
_REST = [c for c in CASES if not (c[0] in _FULL and (c[0] != "BinaryPacked" or c[1] == 128))]


def _device_packed(wv, f, bw, dt, w, rows, cols):
    """Blob packed by the device packer (byte-identical to the reference packer: test_pack_unpack_matvec and
    test_ffn_shapes_full_size) and the oracle's view of the same bytes."""
    q = wv.quant
    blob = q.Pack(q.Format(O.FMT[f]), w, rows, cols, bw, dt)
    ob = O.Blob(O.FMT[f], rows, cols, blob.Raw, blob.Scales, blob.Mins, blob.BlockWeights if f != "none" else 1, dt)
    return blob, ob


@pytest.mark.parametrize("case", _REST, ids=case_id)
@pytest.mark.parametrize("shape", [(4096, 14336), (14336, 4096)], ids=["4096x14336", "14336x4096"])
def test_ffn_shapes_every_layout(wv, case, shape):
    """The benchmark's two shapes for every layout the benchmark times there (the six formats of
    test_ffn_shapes_full_size apart): outputs against the SIMD-path oracle on the benchmark's own inputs."""
    f, bw, dt = case
    rows, cols = shape
    w = np.random.default_rng(2).normal(0, 0.02, rows * cols).astype(np.float32)
    x = np.random.default_rng(1).normal(0, 1, cols).astype(np.float32)
    blob, ob = _device_packed(wv, f, 64 if f == "AffinePacked" else bw, dt, w, rows, cols)
    y = np.zeros(rows, np.float32)
    wv.quant.MatVec(blob, x, y)
    check(y, ob, x, refs=("simd",))


@pytest.mark.parametrize("fmt", ["Q4_K", "Q8_0"])
@pytest.mark.parametrize("shape", [(8192, 8192), (1024, 8192), (28672, 8192), (8192, 28672)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_70b_block_shapes_full_size(wv, fmt, shape):
    """The projection shapes of the 70B decoder block (Q/O 8192x8192, K/V 1024x8192, gate/up 28672x8192,
    down 8192x28672) at full size, weights seed 5."""
    rows, cols = shape
    w = np.random.default_rng(5).normal(0, 0.02, rows * cols).astype(np.float32)
    x = np.random.default_rng(6).normal(0, 1, cols).astype(np.float32)
    blob, ob = _device_packed(wv, fmt, 0, 1, w, rows, cols)
    y = np.zeros(rows, np.float32)
    wv.quant.MatVec(blob, x, y)
    check(y, ob, x, refs=("simd",))


@pytest.mark.parametrize("cols", [8192, 1056, 4608, 17408, 28672])
@pytest.mark.parametrize("fmt", ["Q4_K", "Q5_1", "IQ3_S", "Q8_0"])
def test_kernel_selection_boundaries(wv, fmt, cols):
    """8192 and 4608: TMA-fed kernel with partial column warps; 1056 (cols % 512 != 0), 17408 and
    28672 (more than 16 column warps): register-load kernel with the activation scratch."""
    rows = 97
    w, x = make_w(cols, rows, cols)
    ob = O.pack(fmt, w, rows, cols)
    blob = to_product_blob(wv, ob)
    y = np.zeros(rows, np.float32)
    wv.quant.MatVec(blob, x, y)
    check(y, ob, x)


@pytest.mark.parametrize("fmt", ["Q4_0", "Q4_K", "Q6_K", "IQ1_S", "TernaryPacked", "AffinePacked"])
def test_activation_edge_cases(wv, fmt):
    rows, cols = 64, 4096
    w, x = make_w(31, rows, cols)
    ob = O.pack(fmt, w, rows, cols, 64 if fmt == "AffinePacked" else 0)
    blob = to_product_blob(wv, ob)
    y = np.zeros(rows, np.float32)
    # outliers 1e4 times the typical magnitude, tiny values, an all-zero block, signed zeros
    xo = x.copy()
    xo[[5, 700, 2049]] = [3.0e4, -1.0e4, 2.5e4]
    xo[64:96] = 0.0
    xo[128:160] *= 1e-30
    xo[200] = -0.0
    wv.quant.MatVec(blob, xo, y)
    check(y, ob, xo)
    # zero input gives exactly zero
    wv.quant.MatVec(blob, np.zeros(cols, np.float32), y)
    assert np.all(y == 0)
    # inf / NaN in x poison the outputs (the reference's f32 arithmetic does too) and do not hang
    xn = x.copy()
    xn[10] = np.inf
    wv.quant.MatVec(blob, xn, y)
    assert not np.all(np.isfinite(y))
    from welvet_b200 import _lib
    assert _lib.lib().wv_device_status() == 0


def test_lm_head_slice_row_shard(wv):
    """One rank's 1/8 shard of a 128256x8192 head (16032 rows), Q8_0 and Q4_K: the shard GEMV equals
    the oracle on the same rows."""
    import ctypes as C
    from welvet_b200 import _lib
    L = _lib.lib()
    rows_full, cols, world, rank = 128256, 8192, 8, 3
    lo, hi = C.c_int(), C.c_int()
    _lib.check(L.wv_shard_range(rows_full, rank, world, C.byref(lo), C.byref(hi)))
    n = hi.value - lo.value
    assert n == 16032
    w = np.random.default_rng(5).normal(0, 0.02, n * cols).astype(np.float32)
    x = np.random.default_rng(6).normal(0, 1, cols).astype(np.float32)
    for fmt in ("Q8_0", "Q4_K"):
        blob = wv.quant.Pack(wv.quant.Format(O.FMT[fmt]), w, n, cols)
        ob = O.Blob(O.FMT[fmt], n, cols, blob.Raw, blob.Scales, blob.Mins, blob.BlockWeights)
        y = np.zeros(n, np.float32)
        wv.quant.MatVec(blob, x, y)
        check(y, ob, x, refs=("simd",))


def test_concurrent_host_callers(wv):
    """Callers may be concurrent threads (the reference's goroutines): the synchronous entry serialises
    on its staging buffers and every caller gets its own result."""
    import threading
    rows, cols = 512, 2048
    q = wv.quant
    jobs = []
    for i, f in enumerate(["Q4_K", "Q8_0", "Q4_0", "IQ2_XS"]):
        w, x = make_w(70 + i, rows, cols)
        ob = O.pack(f, w, rows, cols)
        jobs.append((to_product_blob(wv, ob), ob, x))
    for b, _, x in jobs:                       # warm: uploads happen once
        q.MatVec(b, x, np.zeros(rows, np.float32))
    want = [(lambda y: (q.MatVec(b, x, y), y)[1])(np.zeros(rows, np.float32)) for b, _, x in jobs]
    out = [[None] * 20 for _ in jobs]
    errs = []

    def worker(j):
        try:
            b, _, x = jobs[j]
            for k in range(20):
                y = np.zeros(rows, np.float32)
                q.MatVec(b, x, y)
                out[j][k] = y
        except Exception as e:  # noqa: BLE001
            errs.append(e)
    ts = [threading.Thread(target=worker, args=(j,)) for j in range(len(jobs))]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errs, errs
    for j in range(len(jobs)):
        for k in range(20):
            assert np.array_equal(out[j][k].view(np.uint32), want[j].view(np.uint32))
