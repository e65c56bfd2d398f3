"""GPU parity of the decode steps that sit between the projections (RMSNorm, RoPE + cache write,
single-token grouped-query attention, SiLU product, residual add), of the fused projection
epilogues (gate|up with the SiLU product, projection + residual), and of a whole decoder block
in single-token decode with every step on the device — against the oracle's float64 restatements
of the reference's host code."""
import ctypes as C

import numpy as np
import pytest

import oracle as O
from conftest import make_w, to_product_blob

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _dev(t):
    import torch
    return torch.from_numpy(np.ascontiguousarray(t)).cuda()


@pytest.mark.parametrize("rows,dim", [(1, 4096), (3, 8192), (2, 100)])
def test_rmsnorm(wv, rows, dim):
    import torch
    rng = np.random.default_rng(dim)
    x = rng.normal(0, 2, (rows, dim)).astype(np.float32)
    g = rng.normal(1, 0.1, dim).astype(np.float32)
    dx, dg, dy = _dev(x), _dev(g), torch.zeros(rows, dim, device="cuda")
    wv.decode.RMSNormCUDA(dx.data_ptr(), dg.data_ptr(), dy.data_ptr(), rows, dim, 1e-5)
    torch.cuda.synchronize()
    ref = O.rmsnorm(x, g, 1e-5)
    # float64 sum on both sides: the only difference is the order of the additions
    np.testing.assert_allclose(dy.cpu().numpy(), ref, rtol=2e-7, atol=0)


@pytest.mark.parametrize("heads,kv_heads,head_dim,pos", [(32, 8, 128, 2048), (64, 8, 128, 5), (4, 2, 64, 0), (8, 8, 96, 700)])
def test_rope_and_cache_write(wv, heads, kv_heads, head_dim, pos):
    import torch
    rng = np.random.default_rng(pos + heads)
    msl = 512 if pos < 512 else 4096
    q = rng.normal(0, 1, heads * head_dim).astype(np.float32)
    k = rng.normal(0, 1, kv_heads * head_dim).astype(np.float32)
    v = rng.normal(0, 1, kv_heads * head_dim).astype(np.float32)
    ck = torch.zeros(msl, kv_heads * head_dim, device="cuda")
    cv = torch.zeros(msl, kv_heads * head_dim, device="cuda")
    dq, dk, dv = _dev(q), _dev(k), _dev(v)
    wv.decode.RoPECacheCUDA(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ck.data_ptr(), cv.data_ptr(), pos, msl, heads, kv_heads, head_dim, 10000.0)
    torch.cuda.synchronize()
    q_ref = O.rope(q, pos, heads, head_dim).astype(np.float32)
    k_ref = O.rope(k, pos, kv_heads, head_dim).astype(np.float32)
    np.testing.assert_allclose(dq.cpu().numpy(), q_ref, rtol=0, atol=2e-6)
    np.testing.assert_allclose(ck[pos % msl].cpu().numpy(), k_ref, rtol=0, atol=2e-6)
    assert np.array_equal(cv[pos % msl].cpu().numpy(), v)
    assert float(ck.abs().sum()) == pytest.approx(float(np.abs(ck[pos % msl].cpu().numpy()).sum()))   # no other row touched


@pytest.mark.parametrize("heads,kv_heads,head_dim,kv_len,msl", [(32, 8, 128, 2049, 4096), (64, 8, 128, 2049, 2049), (4, 2, 64, 1, 16),
                                                                 (8, 4, 32, 37, 64), (16, 16, 256, 300, 512), (32, 8, 128, 9000, 9000)])
def test_attention_decode(wv, heads, kv_heads, head_dim, kv_len, msl):
    import torch
    rng = np.random.default_rng(kv_len)
    q = rng.normal(0, 1, heads * head_dim).astype(np.float32)
    ck = rng.normal(0, 1, (msl, kv_heads * head_dim)).astype(np.float32)
    cv = rng.normal(0, 1, (msl, kv_heads * head_dim)).astype(np.float32)
    out = torch.full((heads * head_dim,), float("nan"), device="cuda")
    dq, dck, dcv = _dev(q), _dev(ck), _dev(cv)
    for _ in range(2):   # the second call runs on the counters the first one left behind
        wv.decode.AttnDecodeCUDA(dq.data_ptr(), dck.data_ptr(), dcv.data_ptr(), out.data_ptr(), heads, kv_heads, head_dim, kv_len, msl, 1.0 / np.sqrt(head_dim))
        torch.cuda.synchronize()
        ref = O.attn_decode(q, ck, cv, heads, kv_heads, head_dim, kv_len, msl)
        np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=0, atol=2e-5 * max(1.0, float(np.abs(ref).max())))


def test_silu_mul_and_residual_add(wv):
    import torch
    rng = np.random.default_rng(9)
    n = 14336
    g = rng.normal(0, 3, n).astype(np.float32)
    u = rng.normal(0, 1, n).astype(np.float32)
    dg, du, dout = _dev(g), _dev(u), torch.zeros(n, device="cuda")
    wv.decode.SiluMulCUDA(dg.data_ptr(), du.data_ptr(), dout.data_ptr(), n)
    wv.decode.ResidualAddCUDA(dg.data_ptr(), du.data_ptr(), n)
    torch.cuda.synchronize()
    np.testing.assert_allclose(dout.cpu().numpy(), O.silu_mul(g, u), rtol=2e-7, atol=1e-45)
    assert np.array_equal(dg.cpu().numpy(), g + u)


@pytest.mark.parametrize("fmt", ["Q4_K", "Q8_0", "IQ3_S", "none"])
@pytest.mark.parametrize("shape", [(14336, 4096), (300, 512), (28672, 8192), (2048, 28672), (600, 32768)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_fused_swiglu_and_residual_epilogues(wv, fmt, shape):
    """gate|up with the SiLU product in one launch, and projection + residual (also in place), against the
    separate launches of the same kernels (bit for bit where the fused kernel runs) and the oracle."""
    import torch
    from welvet_b200 import _lib
    L = _lib.lib()
    rows, cols = shape
    if fmt == "none" and (rows > 1000 or cols > 28160):
        pytest.skip("FormatNone takes the unfused route (one size is enough); its kernel stages x whole: at most 28160 columns")
    wg, x = make_w(rows + 1, rows, cols)
    wu, _ = make_w(rows + 2, rows, cols)
    obs = [O.pack(fmt, w, rows, cols) for w in (wg, wu)]
    keys = [0x3D0000 + i for i in range(2)]
    for k, ob in zip(keys, obs):
        _lib.check(L.wv_blob_upload(k, ob.format, 1, rows, cols, ob.block_weights, ob.raw.ctypes.data, ob.raw.size,
                                    ob.scales.ctypes.data if ob.scales.size else None, ob.scales.size,
                                    ob.mins.ctypes.data if ob.mins.size else None, ob.mins.size))
    try:
        dx = _dev(x)
        gate, up, h = (torch.zeros(rows, device="cuda") for _ in range(3))
        _lib.check(L.wv_matvec_dev(keys[0], dx.data_ptr(), gate.data_ptr(), 1, cols, rows, None))
        _lib.check(L.wv_matvec_dev(keys[1], dx.data_ptr(), up.data_ptr(), 1, cols, rows, None))
        wv.decode.MatVecSwiGLUCUDA(keys[0], keys[1], dx.data_ptr(), h.data_ptr(), cols, rows)
        torch.cuda.synchronize()
        assert L.wv_device_status() == 0
        g_ref, u_ref = (O.matvec_simd(ob, x, 0) for ob in obs)
        want = O.silu_mul(g_ref, u_ref).astype(np.float64)
        # error budget: each factor is within 1e-3 * sum|w x| of its reference; silu'(g) <= 1.1
        dg, du = (TOL * O.sum_abs_wx(ob, x) for ob in obs)
        bound = 1.1 * dg * np.abs(u_ref) + np.abs(g_ref) * du + dg * du + 1e-6 * np.abs(want) + 1e-30
        assert np.all(np.abs(h.cpu().numpy().astype(np.float64) - want) <= bound)
        # and agrees with the product of the separately computed vectors within the same budget (the separate launches
        # may run on another kernel of the family, with its own rounding)
        sep = O.silu_mul(gate.cpu().numpy(), up.cpu().numpy()).astype(np.float64)
        assert np.all(np.abs(h.cpu().numpy().astype(np.float64) - sep) <= 2 * bound)
        # projection + residual, out of place and in place
        res = np.random.default_rng(3).normal(0, 1, rows).astype(np.float32)
        dres, y = _dev(res), torch.zeros(rows, device="cuda")
        wv.decode.MatVecAddCUDA(keys[0], dx.data_ptr(), dres.data_ptr(), y.data_ptr(), cols, rows)
        wv.decode.MatVecAddCUDA(keys[0], dx.data_ptr(), dres.data_ptr(), dres.data_ptr(), cols, rows)
        torch.cuda.synchronize()
        assert np.all(np.abs(y.cpu().numpy().astype(np.float64) - (g_ref.astype(np.float64) + res)) <= dg + 1e-6 * np.abs(res) + 1e-30)
        assert np.array_equal(y.cpu().numpy(), dres.cpu().numpy())
    finally:
        for k in keys:
            L.wv_blob_evict(k)


@pytest.mark.parametrize("fmt", ["Q4_K", "Q8_0", "IQ4_NL", "none"])
@pytest.mark.parametrize("cols", [4096, 8192, 1000])
def test_rmsnorm_in_the_prologue_of_the_grouped_launch(wv, fmt, cols):
    """Q|K|V on RMSNorm(x) as one launch (the norm in the GEMV's prologue) against the norm's own launch followed by the
    grouped launch, and against the oracle's float64 norm and SIMD-path GEMVs; then gate|up with the SiLU product."""
    import ctypes as C
    import torch
    from welvet_b200 import _lib
    from welvet_b200.decode import MatVecFusedCUDA, RMSNormCUDA
    L = _lib.lib()
    shapes = [(640, cols), (128, cols), (128, cols)]
    obs, keys = [], []
    for i, (r, c) in enumerate(shapes):
        w = make_w(50 + i, r, c)[0]
        ob = O.pack(fmt, w, r, c)
        k = 0x3E0000 + i
        _lib.check(L.wv_blob_upload(k, ob.format, 1, r, c, ob.block_weights, ob.raw.ctypes.data, ob.raw.size,
                                    ob.scales.ctypes.data if ob.scales.size else None, ob.scales.size,
                                    ob.mins.ctypes.data if ob.mins.size else None, ob.mins.size))
        obs.append(ob); keys.append(k)
    try:
        rng = np.random.default_rng(cols)
        x = (rng.normal(0, 3, cols)).astype(np.float32)
        gamma = rng.normal(1, 0.1, cols).astype(np.float32)
        dx, dg = _dev(x), _dev(gamma)
        ys = [torch.full((r,), float("nan"), device="cuda") for r, _ in shapes]
        ka = (C.c_uint64 * 3)(*keys)
        outs = (C.c_int * 3)(*[r for r, _ in shapes])
        MatVecFusedCUDA(ka, dx.data_ptr(), (C.c_void_p * 3)(*[y.data_ptr() for y in ys]), cols, outs, dnorm_gamma=dg.data_ptr(), norm_eps=1e-5)
        xn = torch.zeros(cols, device="cuda")
        RMSNormCUDA(dx.data_ptr(), dg.data_ptr(), xn.data_ptr(), 1, cols, 1e-5)
        refs = [torch.zeros(r, device="cuda") for r, _ in shapes]
        _lib.check(L.wv_matvec_dev_multi(ka, 3, xn.data_ptr(), (C.c_void_p * 3)(*[y.data_ptr() for y in refs]), 1, cols, outs, None))
        torch.cuda.synchronize()
        assert L.wv_device_status() == 0
        xn_ref = O.rmsnorm(x, gamma)
        assert np.max(np.abs(xn.cpu().numpy() - xn_ref)) <= 1e-6 * np.max(np.abs(xn_ref))
        for ob, y, ref in zip(obs, ys, refs):
            want = O.matvec_simd(ob, xn_ref, 0)
            den = O.sum_abs_wx(ob, xn_ref)
            got = y.cpu().numpy().astype(np.float64)
            assert np.all(np.abs(got - want) <= TOL * den + 1e-30)
            # the two device routes differ at most by the rounding of 1 / rms in its last float64 bits
            assert np.all(np.abs(got - ref.cpu().numpy()) <= 2e-6 * den + 1e-30)
        if fmt != "none":
            h = torch.full((shapes[1][0],), float("nan"), device="cuda")
            k2 = (C.c_uint64 * 2)(keys[1], keys[2])
            MatVecFusedCUDA(k2, dx.data_ptr(), (C.c_void_p * 2)(None, h.data_ptr()), cols, (C.c_int * 2)(128, 128), mode=1,
                            dnorm_gamma=dg.data_ptr(), norm_eps=1e-5)
            torch.cuda.synchronize()
            g_ref, u_ref = (O.matvec_simd(ob, xn_ref, 0) for ob in obs[1:])
            want = O.silu_mul(g_ref, u_ref).astype(np.float64)
            dg_, du_ = (TOL * O.sum_abs_wx(ob, xn_ref) for ob in obs[1:])
            bound = 1.1 * dg_ * np.abs(u_ref) + np.abs(g_ref) * du_ + dg_ * du_ + 1e-6 * np.abs(want) + 1e-30
            assert np.all(np.abs(h.cpu().numpy().astype(np.float64) - want) <= bound)
    finally:
        for k in keys:
            L.wv_blob_evict(k)


def test_decoder_block_decode_on_device(wv):
    """The 8B block of the decoder configuration (d_model 4096, 32 / 8 heads of 128, FFN 14336, Q4_K, KV cache of
    2048 positions, RMSNorm eps 1e-5, RoPE theta 10000) decoded for one token entirely on the device, against the
    reference's host arithmetic (oracle float64 steps around the oracle's SIMD-path projections)."""
    import torch
    from welvet_b200 import _lib
    from welvet_b200.decode import BlockConfig, BlockDecoder
    L = _lib.lib()
    d, ffn, n_q, n_kv, hd, ctx = 4096, 14336, 32, 8, 128, 2048
    msl = ctx + 8
    rng = np.random.default_rng(4)
    shapes = {"q": (d, d), "k": (n_kv * hd, d), "v": (n_kv * hd, d), "o": (d, d), "gate": (ffn, d), "up": (ffn, d), "down": (d, ffn)}
    keys, oblobs = {}, {}
    for i, (name, (r, c)) in enumerate(shapes.items()):
        w = rng.normal(0, 0.02, r * c).astype(np.float32)
        b = wv.quant.Pack(wv.quant.Format.FormatQ4_K, w, r, c)
        oblobs[name] = O.Blob(O.FMT["Q4_K"], r, c, b.Raw, b.Scales, b.Mins, b.BlockWeights)
        keys[name] = wv.quant.EnsureResident(b)
        oblobs[name]._keep = b
    kcache = rng.normal(0, 1, (ctx, n_kv * hd)).astype(np.float32)
    vcache = rng.normal(0, 1, (ctx, n_kv * hd)).astype(np.float32)
    x = rng.normal(0, 1, d).astype(np.float32)
    g1 = rng.normal(1, 0.05, d).astype(np.float32)
    g2 = rng.normal(1, 0.05, d).astype(np.float32)
    caches = {n: O.SimdCache(b) for n, b in oblobs.items()}

    def mv(name, vec):
        y = np.zeros(shapes[name][0], np.float32)
        caches[name].matvec(np.ascontiguousarray(vec, np.float32), y, 0)
        return y

    # reference walk (model/transformer/forward.go:57-76, mha/cpu.go:40-240, swiglu/cpu.go:20-62), T = float32
    pos = ctx
    n1 = O.rmsnorm(x, g1)
    q, k, v = mv("q", n1), mv("k", n1), mv("v", n1)
    ck = np.zeros((msl, n_kv * hd)); cv = np.zeros((msl, n_kv * hd))
    ck[:ctx], cv[:ctx] = kcache, vcache
    qr = O.rope(q, pos, n_q, hd)
    ck[pos % msl] = O.rope(k, pos, n_kv, hd)
    cv[pos % msl] = v
    attn = O.attn_decode(qr, ck, cv, n_q, n_kv, hd, pos + 1, msl).astype(np.float32)
    h1 = x + mv("o", attn)
    n2 = O.rmsnorm(h1, g2)
    act = O.silu_mul(mv("gate", n2), mv("up", n2))
    y_ref = h1 + mv("down", act)

    bufs = {"n1": torch.zeros(d, device="cuda"), "q": torch.zeros(n_q * hd, device="cuda"), "k": torch.zeros(n_kv * hd, device="cuda"),
            "v": torch.zeros(n_kv * hd, device="cuda"), "attn": torch.zeros(n_q * hd, device="cuda"), "n2": torch.zeros(d, device="cuda"),
            "ffn": torch.zeros(ffn, device="cuda"), "attn_norm": _dev(g1), "ffn_norm": _dev(g2),
            "cache_k": torch.zeros(msl, n_kv * hd, device="cuda"), "cache_v": torch.zeros(msl, n_kv * hd, device="cuda")}
    bufs["cache_k"][:ctx] = _dev(kcache)
    bufs["cache_v"][:ctx] = _dev(vcache)
    dec = BlockDecoder(BlockConfig(d, n_q, n_kv, hd, ffn, msl), keys, {n: t.data_ptr() for n, t in bufs.items()})
    h = _dev(x)
    dec.step(h.data_ptr(), pos)
    torch.cuda.synchronize()
    assert L.wv_device_status() == 0
    y_dev = h.cpu().numpy()
    assert np.max(np.abs(bufs["attn"].cpu().numpy() - attn)) <= 2e-3 * np.max(np.abs(attn))
    assert np.max(np.abs(y_dev - y_ref)) <= 2e-3 * np.max(np.abs(y_ref))
    # a second token continues from the updated cache without touching the host
    dec.step(h.data_ptr(), pos + 1)
    torch.cuda.synchronize()
    assert L.wv_device_status() == 0 and np.all(np.isfinite(h.cpu().numpy()))
