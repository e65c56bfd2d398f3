"""CPU tests of the oracle itself: hand-derived known-answer blocks (they pin the wire layout
and the dequant formulas against the reference's source text), the bit-for-bit agreement of
the C restatement with the second numpy restatement, internal consistency of the scalar and
SIMD-path arithmetic, the wire round trip, and the committed golden fixtures."""
import os
import struct
import sys

import numpy as np
import pytest

import oracle as O
from oracle import oracle_np as N
from conftest import CASES, case_id, case_ok, make_w

GOLD = os.path.join(os.path.dirname(__file__), "golden", "golden_small.npz")


def f32b(v):
    return struct.pack("<f", v)


# ---------------------------------------------------------------- known-answer blocks
def test_kat_q4_0():
    # maxAbs = 7 -> scale 1; codes are the weights; nibble j of byte j/2 (quant/q4_0.go:23-34)
    w = np.array([(-7 + (i % 15)) for i in range(32)], np.float32)
    b = O.pack("Q4_0", w, 1, 32)
    q = [int(v) & 0xF for v in w]
    exp = f32b(1.0) + bytes(q[2 * j] | (q[2 * j + 1] << 4) for j in range(16))
    assert b.raw.tobytes() == exp
    assert np.array_equal(O.unpack(b), w)


def test_kat_q4_1_q5_and_q8():
    w = np.array([i % 16 for i in range(32)], np.float32)          # mn 0, mx 15 -> scale 1
    b = O.pack("Q4_1", w, 1, 32)
    q = [int(v) for v in w]
    assert b.raw.tobytes() == f32b(1.0) + f32b(0.0) + bytes(q[2 * j] | (q[2 * j + 1] << 4) for j in range(16))
    w5 = np.array([(i % 31) - 15 for i in range(32)], np.float32)  # maxAbs 15 -> scale 1, code = w + 16
    b5 = O.pack("Q5_0", w5, 1, 32)
    bits = 0
    for j, v in enumerate(w5):
        bits |= (int(v) + 16) << (5 * j)
    assert b5.raw.tobytes() == f32b(1.0) + bits.to_bytes(20, "little")
    assert np.array_equal(O.unpack(b5), w5)
    w8 = np.array([127 - 8 * i for i in range(32)], np.float32)    # maxAbs 127 -> scale 1
    b8 = O.pack("Q8_0", w8, 1, 32)
    assert b8.raw.tobytes() == f32b(1.0) + np.array(w8, np.int8).tobytes()


def test_kat_q4_k_and_q6_k():
    # each group of 16 is 0..15: mn 0, sc 1 -> d 1, dmin 0 -> 1, scale byte 255, min byte 0
    w = np.tile(np.arange(16, dtype=np.float32), 16)
    b = O.pack("Q4_K", w, 1, 256)
    nib = [int(v) for v in w]
    exp = f32b(1.0) + f32b(1.0) + bytes([255] * 16) + bytes([0] * 16) + bytes(nib[2 * j] | (nib[2 * j + 1] << 4) for j in range(128))
    assert b.raw.tobytes() == exp and len(exp) == 168
    assert np.array_equal(O.unpack(b), w)
    # Q6_K: amax 31 -> sc 31/32, code = round(w/sc) + 32 (quant/kquant.go:109-123); no mins plane
    w6 = np.tile(np.linspace(-31, 31, 16, dtype=np.float32), 16)
    b6 = O.pack("Q6_K", w6, 1, 256)
    assert b6.raw.size == 216 and b6.raw[:8].tobytes() == f32b(np.float32(31) / np.float32(32)) + f32b(0.0)
    assert bytes(b6.raw[8:24]) == bytes([255] * 16)


def test_kat_bitnet_and_affine():
    w = np.array([1, -1, 0.2, 1, -1, 1, -0.1, -1] * 2, np.float32)  # mean|w| = 0.7875 -> codes 2,0,1,...
    b = O.pack("TernaryPacked", w, 1, 16)
    codes = [2, 0, 1, 2, 0, 2, 1, 0] * 2
    assert struct.unpack("<I", b.raw.tobytes())[0] == sum(c << (2 * j) for j, c in enumerate(codes))
    assert b.scales[0] == np.float32(np.float32(12.6) / np.float32(16)) or abs(b.scales[0] - 0.7875) < 1e-6
    wb = np.array([(-1) ** i * (1 + i) for i in range(32)], np.float32)
    bb = O.pack("BinaryPacked", wb, 1, 32)
    assert struct.unpack("<I", bb.raw.tobytes())[0] == 0x55555555
    wa = np.tile(np.arange(16, dtype=np.float32), 4) * 2 + 3          # mn 3, mx 33, s 2, code = i
    ba = O.pack("AffinePacked", wa, 1, 64)
    assert ba.scales[0] == 2 and ba.mins[0] == 3 and struct.unpack("<I", ba.raw[:4].tobytes())[0] == 0x76543210
    assert np.array_equal(O.unpack(ba), wa)


def test_kat_iq_and_codecs():
    w = np.array([-1.5, -0.5, 0.5, 1.5] * 8, np.float32)              # IQ2: amax 1.5 -> scale 1, code = w + 1.5
    b = O.pack("IQ2_XXS", w, 1, 32)
    assert b.scales[0] == 1 and b.raw.tobytes() == bytes([0b11100100] * 8)
    assert np.array_equal(O.unpack(b), w)
    # Float32ToFloat16 truncates and flushes (core/floatconv.go:6-18)
    v = np.array([1.0, 1.0009765625 + 2 ** -12, 6e-8, 70000.0, -2.5], np.float32)
    assert N.f16_trunc(v).tolist() == [0x3C00, 0x3C01, 0x0000, 0x7C00, 0xC100]
    blob = O.pack("none", v, 1, 5, 0, O.DT_F16)
    assert blob.raw.view(np.uint16).tolist() == [0x3C00, 0x3C01, 0x0000, 0x7C00, 0xC100]
    assert N.bf16_trunc(np.array([1.00390625 + 2 ** -10], np.float32)).tolist() == [0x3F80]


# ---------------------------------------------------------------- two restatements agree
SHAPES = [(4, 256), (3, 100), (1, 31), (7, 512), (2, 1000), (16, 384)]


@pytest.mark.parametrize("case", [c for c in CASES if c[0] != "none"], ids=case_id)
def test_c_and_numpy_restatements_agree(case):
    f, bw, dt = case
    for seed, (rows, cols) in enumerate(SHAPES):
        if not case_ok(case, rows, cols):
            continue
        w, x = make_w(seed, rows, cols)
        if seed == 3:
            w[0, :40] = 0
        b = O.pack(f, w, rows, cols, bw)
        raw, sc, mn = N.pack(f, w, rows, cols, bw)
        assert np.array_equal(b.raw, raw)
        assert np.array_equal(b.scales.view(np.uint32), np.asarray(sc, np.float32).view(np.uint32))
        assert np.array_equal(b.mins.view(np.uint32), np.asarray(mn, np.float32).view(np.uint32))
        u1 = O.unpack(b)
        u2 = N.unpack(f, rows, cols, b.raw, b.scales, b.mins, b.block_weights)
        assert np.array_equal(u1.view(np.uint32), u2.view(np.uint32))


@pytest.mark.parametrize("case", CASES, ids=case_id)
def test_scalar_simd_paths_consistent(case):
    f, bw, dt = case
    rows, cols = 70, 512
    w, x = make_w(5, rows, cols)
    b = O.pack(f, w, rows, cols, bw, dt)
    y_s, y_1, y_4 = O.matvec(b, x), O.matvec_simd(b, x, 1), O.matvec_simd(b, x, 4)
    assert np.array_equal(y_1, y_4), "row sharding over threads must not change results"
    den = O.sum_abs_wx(b, x)
    assert np.all(np.abs(y_s.astype(np.float64) - y_1) <= 1e-5 * den + 1e-30)
    O.lib().wvo_force_scalar(1)
    try:
        assert np.array_equal(O.matvec_simd(b, x, 1), y_1), "AVX2 and scalar-order block dots differ"
    finally:
        O.lib().wvo_force_scalar(0)


@pytest.mark.parametrize("case", [c for c in CASES if c[0] != "none"], ids=case_id)
def test_wire_round_trip(case):
    f, bw, dt = case
    rows, cols = 6, 256
    w, _ = make_w(9, rows, cols)
    b = O.pack(f, w, rows, cols, bw)
    wire = O.wire_encode(b)
    assert wire.size == 12 + b.packed_bytes
    ns, nm, nr = struct.unpack("<III", wire[:12].tobytes())
    assert (ns, nm, nr) == (b.scales.size, b.mins.size, b.raw.size)
    d = O.wire_decode(f, rows, cols, wire)
    assert np.array_equal(d.raw, b.raw) and np.array_equal(d.scales, b.scales) and np.array_equal(d.mins, b.mins)
    if f == "BinaryPacked":
        assert d.block_weights == (128 if bw == 128 else 32)  # InferBinaryBlockWeights
        assert np.array_equal(O.unpack(d), O.unpack(b))


def test_golden_fixtures():
    g = np.load(GOLD)
    for rows, cols in ((8, 512), (3, 100)):
        w, x = g[f"w_{rows}x{cols}"], g[f"x_{rows}x{cols}"]
        for c in CASES:
            if not case_ok(c, rows, cols):
                continue
            f, bw, dt = c
            k = f"{case_id(c)}_{rows}x{cols}"
            b = O.pack(f, w, rows, cols, bw, dt)
            assert np.array_equal(b.raw, g[k + "_raw"]), k
            assert np.array_equal(b.scales, g[k + "_scales"]) and np.array_equal(b.mins, g[k + "_mins"]), k
            assert np.array_equal(O.unpack(b).view(np.uint32), g[k + "_unpack"].view(np.uint32)), k
            assert np.array_equal(O.matvec(b, x), g[k + "_y_scalar"]), k


def test_argmax_restatement():
    """sampling.ArgMax: first strict maximum; NaN never wins; NaN in position 0 keeps index 0; empty -> 0."""
    assert O.argmax(np.array([1, 3, 3, 2], np.float32)) == 1
    assert O.argmax(np.array([np.nan, 3, 3, 2], np.float32)) == 0
    assert O.argmax(np.array([1, np.nan, 0.5], np.float32)) == 0
    assert O.argmax(np.array([-np.inf, -np.inf], np.float32)) == 0
    assert O.argmax(np.zeros(0, np.float32)) == 0
    v = np.random.default_rng(0).normal(0, 1, 5000).astype(np.float32)
    assert O.argmax(v) == int(np.argmax(v))


def test_oracle_against_reference_dump():
    """Pins the oracle against the reference itself when tests/golden/ref_go_dump.bin is present: the
    output of oracle/ref_dump/main.go (the reference's own quant.Pack / Unpack / MatVec and
    dense.MatVecPackedBlob run with Go on the inputs of tests/golden/make_ref_inputs.py). Packed
    bytes, scales, mins and dequantised weights must agree bit for bit, the scalar MatVec bit for bit
    (same f32 order), the SIMD path to 1e-6 relative (f64 accumulation, thread split may differ)."""
    import struct
    gold = os.path.join(os.path.dirname(__file__), "golden")
    dump = os.path.join(gold, "ref_go_dump.bin")
    if not os.path.exists(dump):
        pytest.skip("parity unpinned: reference fixtures absent (no Go toolchain here; see oracle/ref_dump/main.go)")
    sys.path.insert(0, gold)
    import make_ref_inputs
    data = open(dump, "rb").read()
    (n,) = struct.unpack_from("<I", data, 0)
    off = 4
    cs = list(make_ref_inputs.cases())
    assert n == len(cs)
    for f, rows, cols, w, x in cs:
        fmt, r, c, bw, nraw, ns, nm, has_simd = struct.unpack_from("<8I", data, off)
        off += 32
        assert (fmt, r, c) == (f, rows, cols)
        raw = np.frombuffer(data, np.uint8, nraw, off); off += nraw
        scales = np.frombuffer(data, "<f4", ns, off); off += 4 * ns
        mins = np.frombuffer(data, "<f4", nm, off); off += 4 * nm
        un = np.frombuffer(data, "<f4", rows * cols, off); off += 4 * rows * cols
        y_scalar = np.frombuffer(data, "<f4", rows, off); off += 4 * rows
        y_simd = np.frombuffer(data, "<f4", rows, off); off += 4 * rows
        ob = O.pack(f, w, rows, cols, 64 if f == O.FMT["AffinePacked"] else 0)
        tag = f"{O.FORMATS[f]} {rows}x{cols}"
        assert np.array_equal(ob.raw, raw), tag + ": Raw"
        assert np.array_equal(ob.scales.view(np.uint32), scales.view(np.uint32)), tag + ": Scales"
        assert np.array_equal(ob.mins.view(np.uint32), mins.view(np.uint32)), tag + ": Mins"
        assert np.array_equal(O.unpack(ob).view(np.uint32), un.view(np.uint32)), tag + ": Unpack"
        assert np.array_equal(O.matvec(ob, x).view(np.uint32), y_scalar.view(np.uint32)), tag + ": MatVec"
        if has_simd:
            np.testing.assert_allclose(O.matvec_simd(ob, x, 1), y_simd, rtol=1e-6, atol=1e-7, err_msg=tag + ": SIMD path")
    assert off == len(data)


def test_topk_restatement_known_answers():
    """sampling.SampleTopK by hand: logits (0, ln 2, ln 4, -9) at temperature 1, top 3 -> weights 1, 1/2, 1/4 in the
    order index 2, 1, 0 (sum 1.75); the draw u * 1.75 falls in [0, 1] -> 2, (1, 1.5] -> 1, (1.5, 1.75] -> 0."""
    v = np.array([0.0, np.log(2.0), np.log(4.0), -9.0], np.float32)
    assert O.topk_sample(v, 3, 1.0, False, 0.0) == 2
    assert O.topk_sample(v, 3, 1.0, False, 1.0 / 1.75 - 1e-9) == 2
    assert O.topk_sample(v, 3, 1.0, False, 1.0 / 1.75 + 1e-6) == 1
    assert O.topk_sample(v, 3, 1.0, False, 1.5 / 1.75 + 1e-6) == 0
    assert O.topk_sample(v, 3, 1.0, False, 1.0) == 0
    assert O.topk_sample(v, 0, 1.0, False, 1.0) == 3          # top_k <= 0: every logit is a candidate
    assert O.topk_sample(v, 9, 1.0, False, 1.0) == 3          # top_k >= n as well
    for args in ((1, 1.0, False), (3, 0.0, False), (3, -1.0, False), (3, 1.0, True)):   # the greedy short-cuts
        assert O.topk_sample(v, *args, 0.9) == 2
    assert O.topk_sample(np.zeros(0, np.float32), 3, 1.0, False, 0.5) == 0
    t = np.array([1, 5, 5, 5, 2], np.float32)                 # equal values go by rising index here
    assert [O.topk_sample(t, 2, 1.0, False, u) for u in (0.1, 0.9)] == [1, 2]
    # temperature divides in float32 before the ordering: a high temperature flattens the weights
    hot = [O.topk_sample(v, 3, 100.0, False, u) for u in (0.2, 0.5, 0.9)]
    assert hot == [2, 1, 0]


@pytest.mark.parametrize("case", CASES, ids=case_id)
def test_decode_row_restatement_equals_unpack_rows(case):
    f, bw, dt = case
    if f == "none":
        pytest.skip("quant.DecodeRow refuses FormatNone")
    rows, cols = (9, 256) if (f == "AffinePacked" or bw == 128) else (9, 200)
    w = np.random.default_rng(11).normal(0, 0.02, rows * cols).astype(np.float32)
    ob = O.pack(f, w, rows, cols, bw, dt)
    full = O.unpack(ob).reshape(rows, cols)
    for r in range(rows):
        assert O.decode_row(ob, r).tobytes() == full[r].tobytes()
    with pytest.raises(ValueError):
        O.decode_row(ob, rows)
