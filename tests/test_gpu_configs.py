"""GPU parity for the remaining benchmark configurations: the small-batch variant
(M in {1, 4, 16, 64, 256} rows of activations against a 4096x4096 matrix in Q8_0 and the 4-bit
k-quant) and one Llama-style decoder block in single-token decode where only the seven
projections run on the device."""
import numpy as np
import pytest

import oracle as O
from conftest import to_product_blob

pytestmark = pytest.mark.gpu
TOL = 1e-3


@pytest.mark.parametrize("fmt", ["Q8_0", "Q4_K"])
def test_small_batch_variant(wv, fmt):
    rows = cols = 4096
    rng = np.random.default_rng(3)
    w = rng.normal(0, 0.02, rows * cols).astype(np.float32)
    blob = wv.quant.Pack(wv.quant.Format(O.FMT[fmt]), w, rows, cols)
    ob = O.Blob(O.FMT[fmt], rows, cols, blob.Raw, blob.Scales, blob.Mins, blob.BlockWeights)
    st = wv.weights.FromBlob(blob)
    layer = wv.dense.Layer(cols, rows, wv.dense.ActivationLinear, st)
    cache = O.SimdCache(ob)
    for m in (1, 4, 16, 64, 256):
        X = rng.normal(0, 0.02, (m, cols)).astype(np.float32)
        pre, post = wv.dense.Forward(layer, X)
        assert pre.shape == (m, rows)
        for i in sorted(set([0, m // 2, m - 1])):
            ref = np.zeros(rows, np.float32)
            cache.matvec(X[i], ref, 0)
            den = O.sum_abs_wx(ob, X[i])
            assert np.all(np.abs(pre[i].astype(np.float64) - ref) <= TOL * den + 1e-30), (fmt, m, i)


def _rmsnorm(x, eps=1e-5):
    x = x.astype(np.float64)
    return (x / np.sqrt(np.mean(x * x) + eps)).astype(np.float32)


def _rope(v, pos, head_dim, theta=10000.0):
    v = v.astype(np.float64).reshape(-1, head_dim)
    half = head_dim // 2
    inv = theta ** (-np.arange(half) * 2.0 / head_dim)
    ang = pos * inv
    c, s = np.cos(ang), np.sin(ang)
    a, b = v[:, :half], v[:, half:]
    return np.concatenate([a * c - b * s, a * s + b * c], axis=1).reshape(-1)


def _block(matvec, P, x, kcache, vcache, pos, n_q=32, n_kv=8, hd=128):
    """One decoder block in single-token decode; `matvec(name, vec)` does the projections,
    everything else is host f64 arithmetic (as the reference's mha / swiglu host paths)."""
    h = _rmsnorm(x)
    q, k, v = matvec("q", h), matvec("k", h), matvec("v", h)
    q = _rope(q, pos, hd)
    k = _rope(k, pos, hd)
    K = np.concatenate([kcache, k.reshape(1, -1)], axis=0).reshape(-1, n_kv, hd)
    V = np.concatenate([vcache, v.astype(np.float64).reshape(1, -1)], axis=0).reshape(-1, n_kv, hd)
    out = np.zeros(n_q * hd)
    for hq in range(n_q):
        g = hq // (n_q // n_kv)
        sc = K[:, g, :] @ q[hq * hd:(hq + 1) * hd] / np.sqrt(hd)
        p = np.exp(sc - sc.max()); p /= p.sum()
        out[hq * hd:(hq + 1) * hd] = p @ V[:, g, :]
    x1 = x.astype(np.float64) + matvec("o", out.astype(np.float32))
    h2 = _rmsnorm(x1.astype(np.float32))
    gate, up = matvec("gate", h2).astype(np.float64), matvec("up", h2).astype(np.float64)
    act = (gate / (1.0 + np.exp(-gate))) * up
    return x1 + matvec("down", act.astype(np.float32)), {"q_in": h, "o_in": out.astype(np.float32), "ffn_in": h2, "down_in": act.astype(np.float32)}


def test_decoder_block_single_token_decode(wv):
    d, ffn, n_kv, hd, ctx = 4096, 14336, 8, 128, 2048
    rng = np.random.default_rng(4)
    shapes = {"q": (d, d), "k": (n_kv * hd, d), "v": (n_kv * hd, d), "o": (d, d), "gate": (ffn, d), "up": (ffn, d), "down": (d, ffn)}
    blobs, oblobs = {}, {}
    for name, (r, c) in shapes.items():
        w = rng.normal(0, 0.02, r * c).astype(np.float32)
        blobs[name] = wv.quant.Pack(wv.quant.Format.FormatQ4_K, w, r, c)
        b = blobs[name]
        oblobs[name] = O.Blob(O.FMT["Q4_K"], r, c, b.Raw, b.Scales, b.Mins, b.BlockWeights)
    kcache = rng.normal(0, 1, (ctx, n_kv * hd))
    vcache = rng.normal(0, 1, (ctx, n_kv * hd))
    x = rng.normal(0, 1, d).astype(np.float32)
    caches = {n: O.SimdCache(b) for n, b in oblobs.items()}

    def mv_dev(name, vec):
        y = np.zeros(shapes[name][0], np.float32)
        wv.dense.MatVecPackedBlob(blobs[name], np.ascontiguousarray(vec, np.float32), y)
        return y

    def mv_ref(name, vec):
        y = np.zeros(shapes[name][0], np.float32)
        caches[name].matvec(np.ascontiguousarray(vec, np.float32), y, 0)
        return y

    y_ref, ins = _block(mv_ref, None, x, kcache, vcache, ctx)
    y_dev, _ = _block(mv_dev, None, x, kcache, vcache, ctx)
    # every projection, fed the reference's own intermediate activations, is within tolerance
    for name, key in (("q", "q_in"), ("k", "q_in"), ("v", "q_in"), ("o", "o_in"), ("gate", "ffn_in"), ("up", "ffn_in"), ("down", "down_in")):
        den = O.sum_abs_wx(oblobs[name], ins[key])
        err = np.abs(mv_dev(name, ins[key]).astype(np.float64) - mv_ref(name, ins[key]))
        assert np.all(err <= TOL * den + 1e-30), name
    # and the block output agrees end to end
    assert np.max(np.abs(y_dev - y_ref)) <= 2e-3 * np.max(np.abs(y_ref))


@pytest.mark.parametrize("fmt", ["Q8_0", "Q4_K"])
def test_lm_head_shape(wv, fmt):
    """The largest single matrix of the configurations: an LM head of 128256 x 8192 (1.05 G weights,
    1.18 GB in Q8_0). Packed on the device, multiplied on the device, checked against the restated
    SIMD path on every row; the same blob split into 8 row shards must reassemble to the same y."""
    import ctypes as C
    rows, cols = 128256, 8192
    rng = np.random.default_rng(5)
    w = rng.standard_normal(rows * cols, dtype=np.float32)
    w *= np.float32(0.02)
    x = rng.standard_normal(cols, dtype=np.float32)
    blob = wv.quant.Pack(wv.quant.Format(O.FMT[fmt]), w, rows, cols)
    del w
    y = np.zeros(rows, np.float32)
    wv.dense.MatVecPackedBlob(blob, x, y)
    ob = O.Blob(O.FMT[fmt], rows, cols, blob.Raw, blob.Scales, blob.Mins, blob.BlockWeights)
    ref = O.matvec_simd(ob, x, 0)
    den = O.sum_abs_wx(ob, x)
    err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
    assert np.all(err <= TOL * den + 1e-30), float(np.max(err / np.maximum(den, 1e-30)))
    # 8 row shards (16032 rows each), each computed on its own, give back the same vector
    L = wv._lib.lib()
    import torch
    dx = torch.from_numpy(x).cuda()
    dy = torch.zeros(rows, device="cuda")
    world = 8
    for r in range(world):
        key = 0xB20000 + r
        wv._lib.check(L.wv_blob_upload_shard(key, O.FMT[fmt], 1, rows, cols, blob.BlockWeights, blob.Raw.ctypes.data, blob.Raw.size,
                                             None, 0, None, 0, r, world))
        r0, r1 = C.c_int(), C.c_int()
        wv._lib.check(L.wv_shard_range(rows, r, world, C.byref(r0), C.byref(r1)))
        wv._lib.check(L.wv_matvec_dev(key, dx.data_ptr(), dy.data_ptr() + 4 * r0.value, 1, cols, r1.value - r0.value, None))
        torch.cuda.synchronize()
        L.wv_blob_evict(key)
    assert np.array_equal(dy.cpu().numpy().view(np.uint32), y.view(np.uint32))
