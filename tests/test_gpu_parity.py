"""GPU parity: the CUDA path through the C ABI against the CPU oracle on identical inputs.

Bars: packed bytes and dequantised weights bit-exact; outputs |y - y_ref| <= 1e-3 * sum|w x|
per row (the tolerance the backend is specified to), against both reference arithmetics —
the scalar f32 quant.MatVec and the f64 SIMD path."""
import numpy as np
import pytest

import oracle as O
from conftest import CASES, case_id, case_ok, make_w, to_product_blob

pytestmark = pytest.mark.gpu
TOL = 1e-3

SHAPES = [(8, 256), (64, 512), (33, 1024), (5, 96), (3, 100), (1, 31), (130, 4096)]


def _check_y(y, ob, x):
    den = O.sum_abs_wx(ob, x)
    for name, ref in (("scalar", O.matvec(ob, x)), ("simd", O.matvec_simd(ob, x, 1))):
        if name == "simd" and ob.cols % 32 != 0:
            continue  # the reference's SIMD drivers are only defined for 32-aligned rows
        err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
        bad = err > TOL * den + 1e-30
        assert not bad.any(), f"{name}: {bad.sum()} rows out of tolerance, worst ratio {np.max(err / np.maximum(den, 1e-30)):.3e}"


@pytest.mark.parametrize("case", CASES, ids=case_id)
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
def test_pack_unpack_matvec(wv, case, shape):
    rows, cols = shape
    if not case_ok(case, rows, cols):
        pytest.skip("layout needs aligned cols")
    f, bw, dt = case
    w, x = make_w(rows * 131 + cols, rows, cols)
    if rows >= 8:
        w[1, : min(cols, 64)] = 0.0  # an all-zero block
        w[2, :] = 0.0                # an all-zero row: tolerance is exactly 0 for symmetric formats
    ob = O.pack(f, w, rows, cols, bw, dt)
    q = wv.quant
    # device packer == reference packer, byte for byte
    pb = q.Pack(q.Format(ob.format), w, rows, cols, bw, dt)
    assert np.array_equal(pb.Raw, ob.raw), "packed Raw differs"
    assert np.array_equal(pb.Scales.view(np.uint32), ob.scales.view(np.uint32)), "Scales differ"
    assert np.array_equal(pb.Mins.view(np.uint32), ob.mins.view(np.uint32)), "Mins differ"
    # dequantised weights bit-exact
    blob = to_product_blob(wv, ob)
    got = q.Unpack(blob)
    assert np.array_equal(got.view(np.uint32), O.unpack(ob).view(np.uint32)), "dequantised weights differ"
    # GEMV within tolerance
    y = np.zeros(rows, np.float32)
    wv.dense.MatVecPackedBlob(blob, x, y)
    _check_y(y, ob, x)


@pytest.mark.parametrize("case", [c for c in CASES if c[0] in ("Q4_K", "Q8_0", "Q4_0", "IQ3_S", "none")], ids=case_id)
def test_batch_forward(wv, case):
    f, bw, dt = case
    rows, cols, batch = 96, 512, 5
    w, _ = make_w(7, rows, cols)
    X = np.random.default_rng(8).normal(0, 1, (batch, cols)).astype(np.float32)
    ob = O.pack(f, w, rows, cols, bw, dt)
    st = wv.weights.FromBlob(to_product_blob(wv, ob))
    layer = wv.dense.Layer(cols, rows, wv.dense.ActivationLinear, st)
    pre, post = wv.dense.Forward(layer, X)
    assert pre is post and pre.shape == (batch, rows)
    for b in range(batch):
        _check_y(pre[b], ob, X[b])
    # bias + activation applied after the GEMV
    st.Bias = np.linspace(-1, 1, rows)
    layer.Activation = wv.dense.ActivationReLU
    pre2, post2 = wv.dense.Forward(layer, X)
    np.testing.assert_allclose(pre2, pre + st.Bias.astype(np.float32), rtol=0, atol=1e-6)
    np.testing.assert_array_equal(post2, np.maximum(pre2, 0))


def test_wire_upload_and_cache(wv):
    from welvet_b200 import _lib
    L = _lib.lib()
    rows, cols = 16, 256
    w, x = make_w(3, rows, cols)
    for f, bw in (("Q4_K", 0), ("IQ2_XS", 0), ("BinaryPacked", 128), ("AffinePacked", 64), ("Q5_1", 0)):
        ob = O.pack(f, w, rows, cols, bw)
        wire = O.wire_encode(ob)
        key = 0xABC000 + ob.format * 4 + (1 if bw == 128 else 0)
        before = L.wv_cache_bytes()
        _lib.check(L.wv_blob_upload_wire(key, ob.format, 1, rows, cols, wire.ctypes.data, wire.size))
        assert L.wv_blob_has(key) == 1 and L.wv_cache_bytes() > before
        out = np.empty(rows * cols, np.float32)
        _lib.check(L.wv_unpack(key, out.ctypes.data))
        assert np.array_equal(out.view(np.uint32), O.unpack(ob).view(np.uint32))
        _lib.check(L.wv_blob_evict(key))
        assert L.wv_blob_has(key) == 0 and L.wv_cache_bytes() == before
        assert L.wv_blob_evict(key) == _lib.WV_ENOTFOUND


def test_errors(wv):
    from welvet_b200 import _lib
    L = _lib.lib()
    rows, cols = 8, 256
    w, x = make_w(4, rows, cols)
    ob = O.pack("Q4_0", w, rows, cols)
    blob = to_product_blob(wv, ob)
    y = np.zeros(rows, np.float32)
    with pytest.raises(wv.WelvetError):  # short x
        wv.quant.MatVec(blob, x[:100], y)
    with pytest.raises(wv.WelvetError):  # short y
        wv.quant.MatVec(blob, x, y[:3])
    key = wv.quant.EnsureResident(blob)
    assert L.wv_matvec(key, x.ctypes.data, y.ctypes.data, 1, cols + 32, rows) == _lib.WV_ESHAPE
    assert L.wv_matvec(123456789, x.ctypes.data, y.ctypes.data, 1, cols, rows) == _lib.WV_ENOTFOUND
    # truncated raw, unknown format, unsupported FormatNone dtype
    assert L.wv_blob_upload(1, ob.format, 1, rows, cols, 32, ob.raw.ctypes.data, ob.raw.size - 20, None, 0, None, 0) == _lib.WV_ESHAPE
    assert L.wv_blob_upload(2, 77, 1, rows, cols, 0, ob.raw.ctypes.data, ob.raw.size, None, 0, None, 0) == _lib.WV_EFORMAT
    assert L.wv_blob_upload(3, 0, 9, rows, cols, 0, ob.raw.ctypes.data, ob.raw.size, None, 0, None, 0) == _lib.WV_EFORMAT
    wire = O.wire_encode(O.pack("IQ4_XS", w, rows, cols))
    assert L.wv_blob_upload_wire(4, 17, 1, rows, cols, wire.ctypes.data, wire.size - 5) == _lib.WV_ESHAPE
    # cache budget: the sentinel the reference calls "VRAM budget full"
    L.wv_cache_set_limit(L.wv_cache_bytes() + 16)
    assert L.wv_blob_upload(5, ob.format, 1, rows, cols, 32, ob.raw.ctypes.data, ob.raw.size, None, 0, None, 0) == _lib.WV_ENOMEM
    L.wv_cache_set_limit(0)
    assert b"budget" in L.wv_last_error()


@pytest.mark.parametrize("case", [c for c in CASES if c[0] in ("Q4_K", "Q8_0", "IQ3_XXS", "BinaryPacked", "AffinePacked", "none")], ids=case_id)
def test_row_shards_match_full(wv, case):
    """Each rank's shard of W gives exactly that rank's slice of the single-device y."""
    from welvet_b200 import _lib
    import ctypes as C
    L = _lib.lib()
    f, bw, dt = case
    rows, cols, world = 64, 512, 4
    w, x = make_w(11, rows, cols)
    ob = O.pack(f, w, rows, cols, bw, dt)
    blob = to_product_blob(wv, ob)
    y_full = np.zeros(rows, np.float32)
    wv.dense.MatVecPackedBlob(blob, x, y_full)
    y_cat = np.zeros(rows, np.float32)
    for rank in range(world):
        lo, hi = C.c_int(), C.c_int()
        _lib.check(L.wv_shard_range(rows, rank, world, C.byref(lo), C.byref(hi)))
        key = 0x5A000 + rank
        _lib.check(L.wv_blob_upload_shard(key, ob.format, dt, rows, cols, ob.block_weights, ob.raw.ctypes.data, ob.raw.size,
                                          ob.scales.ctypes.data, ob.scales.size, ob.mins.ctypes.data, ob.mins.size, rank, world))
        part = np.zeros(hi.value - lo.value, np.float32)
        _lib.check(L.wv_matvec(key, x.ctypes.data, part.ctypes.data, 1, cols, hi.value - lo.value))
        y_cat[lo.value:hi.value] = part
        _lib.check(L.wv_blob_evict(key))
    assert np.array_equal(y_cat.view(np.uint32), y_full.view(np.uint32))
