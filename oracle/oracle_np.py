"""Second, independently structured restatement of the reference's Pack / Unpack in numpy.

TEST INFRASTRUCTURE ONLY. The C restatement (welvet_oracle.c) walks blocks one at a time the
way the Go code does; this one works on whole (blocks x width) arrays, builds bit streams
with packbits and decodes them with unpackbits. The two must agree bit for bit on packed
bytes and on dequantised floats — that agreement is what pins the oracle while the
reference binary itself cannot be run. Sources restated (paths inside the reference):
quant/q4_0.go q4_1.go q5_0.go q5_1.go q8_0.go kquant.go iq.go ternary.go binary.go
binary_g128.go affine_pack.go affine_g64.go helpers.go, core/floatconv.go.

Every float32 operation is a separately rounded numpy float32 op (amd64 Go does not fuse).
"""
from __future__ import annotations

import numpy as np

f32 = np.float32
f64 = np.float64

IQ4NL = np.array([-1.0, -0.6961928, -0.52507305, -0.3949175, -0.28444138, -0.18477343,
                  -0.091050036, 0.0, 0.0795803, 0.1609302, 0.2461123, 0.33791524,
                  0.44070983, 0.562617, 0.72295684, 1.0], dtype=f32)

K_SPEC = {"Q2_K": (2, True, 3, 0), "Q3_K": (3, True, 7, 0), "Q4_K": (4, True, 15, 0),
          "Q5_K": (5, True, 31, 0), "Q6_K": (6, False, 63, 32)}
IQ_SPEC = {"IQ1_S": (1, 32, False, 0.5), "IQ2_XXS": (2, 32, False, 1.5), "IQ2_XS": (2, 16, False, 1.5),
           "IQ3_XXS": (3, 32, False, 3.5), "IQ3_S": (3, 16, False, 3.5), "IQ4_NL": (4, 32, True, 0.0),
           "IQ4_XS": (4, 16, False, 7.5)}


def go_round(v):
    """math.Round: half away from zero, on float64."""
    v = np.asarray(v, f64)
    t = np.trunc(v)
    return t + np.sign(v) * (np.abs(v - t) >= 0.5)


def _blocks(w, width):
    """(nblocks, width) view padded by edge replication + validity mask."""
    w = np.asarray(w, f32).reshape(-1)
    n = w.size
    nb = (n + width - 1) // width
    idx = np.arange(nb * width).reshape(nb, width)
    valid = idx < n
    first = np.minimum(idx[:, :1], n - 1)
    blk = w[np.where(valid, idx, first)]
    return blk, valid


def _codes_to_bytes(codes, bits):
    """LSB-first bit stream of `bits`-wide codes (quant/helpers.go bitWriter)."""
    codes = np.asarray(codes, np.uint32).reshape(-1, 1)
    bitsarr = ((codes >> np.arange(bits, dtype=np.uint32)) & 1).astype(np.uint8).reshape(-1)
    return np.packbits(bitsarr, bitorder="little")


def _bytes_to_codes(buf, bits, count):
    bitsarr = np.unpackbits(np.asarray(buf, np.uint8), bitorder="little")
    need = bits * count
    if bitsarr.size < need:
        bitsarr = np.concatenate([bitsarr, np.zeros(need - bitsarr.size, np.uint8)])
    b = bitsarr[:need].reshape(count, bits).astype(np.uint32)
    return (b << np.arange(bits, dtype=np.uint32)).sum(axis=1).astype(np.uint32)


def _max_abs(blk, valid):
    return np.max(np.where(valid, np.abs(blk), f32(0)), axis=1).astype(f32)


def _min_max(blk):
    return blk.min(axis=1).astype(f32), blk.max(axis=1).astype(f32)


def _abs_mean(blk, valid):
    s = np.zeros(blk.shape[0], f32)
    for j in range(blk.shape[1]):
        s = (s + np.where(valid[:, j], np.abs(blk[:, j]), f32(0))).astype(f32)
    cnt = valid.sum(axis=1).astype(f32)
    return (s / cnt).astype(f32)


def _one_if_zero(s):
    return np.where(s == 0, f32(1), s).astype(f32)


def _f32_bytes(a):
    return np.ascontiguousarray(a, f32).view(np.uint8).reshape(a.shape[0], -1)


# ---------------------------------------------------------------- pack
def pack(fmt: str, w, rows: int, cols: int, block_weights: int = 0):
    """Returns (raw uint8, scales f32, mins f32)."""
    w = np.asarray(w, f32).reshape(-1)[: rows * cols]
    e = np.zeros(0, f32)
    if fmt == "Q4_0":
        blk, valid = _blocks(w, 32)
        scale = _one_if_zero((_max_abs(blk, valid) / f32(7)).astype(f32))
        q = go_round((blk / scale[:, None]).astype(f32).astype(f64))
        q = np.where(valid, np.clip(q, -8, 7), 0).astype(np.int64) & 0xF
        nib = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
        return np.concatenate([_f32_bytes(scale), nib], axis=1).reshape(-1), e, e
    if fmt == "Q4_1":
        blk, valid = _blocks(w, 32)
        mn, mx = _min_max(blk)
        scale = _one_if_zero(((mx - mn).astype(f32) / f32(15)).astype(f32))
        q = go_round((((blk - mn[:, None]).astype(f32)) / scale[:, None]).astype(f32).astype(f64))
        q = np.where(valid, np.clip(q, 0, 15), 0).astype(np.int64)
        nib = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
        return np.concatenate([_f32_bytes(scale), _f32_bytes(mn), nib], axis=1).reshape(-1), e, e
    if fmt in ("Q5_0", "Q5_1"):
        blk, valid = _blocks(w, 32)
        if fmt == "Q5_0":
            scale = _one_if_zero((_max_abs(blk, valid) / f32(15)).astype(f32))
            q = go_round(blk.astype(f64) / scale.astype(f64)[:, None]) + 16
            q = np.where(valid, np.clip(q, 0, 31), 16).astype(np.uint32)
            head = _f32_bytes(scale)
        else:
            mn, mx = _min_max(blk)
            scale = _one_if_zero(((mx - mn).astype(f32) / f32(31)).astype(f32))
            q = go_round((((blk - mn[:, None]).astype(f32)) / scale[:, None]).astype(f32).astype(f64))
            q = np.where(valid, np.clip(q, 0, 31), 0).astype(np.uint32)
            head = np.concatenate([_f32_bytes(scale), _f32_bytes(mn)], axis=1)
        stream = _codes_to_bytes(q, 5).reshape(-1, 20)
        return np.concatenate([head, stream], axis=1).reshape(-1), e, e
    if fmt == "Q8_0":
        blk, valid = _blocks(w, 32)
        scale = _one_if_zero((_max_abs(blk, valid) / f32(127)).astype(f32))
        q = go_round(blk.astype(f64) / scale.astype(f64)[:, None])
        q = np.where(valid, np.clip(q, -127, 127), 0).astype(np.int8).view(np.uint8)
        return np.concatenate([_f32_bytes(scale), q], axis=1).reshape(-1), e, e
    if fmt in K_SPEC:
        bits, has_dmin, qmax, mid = K_SPEC[fmt]
        n = w.size
        grp, valid = _blocks(w, 16)
        nsb = (n + 255) // 256
        ng = nsb * 16
        if grp.shape[0] < ng:  # groups that start past n
            pad = ng - grp.shape[0]
            grp = np.concatenate([grp, np.zeros((pad, 16), f32)])
            valid = np.concatenate([valid, np.zeros((pad, 16), bool)])
        live = valid[:, 0]
        if has_dmin:
            gmn, gmx = _min_max(np.where(valid, grp, grp[:, :1]))
            sc = _one_if_zero(((gmx - gmn).astype(f32) / f32(qmax)).astype(f32))
            q = go_round((((grp - gmn[:, None]).astype(f32)) / sc[:, None]).astype(f32).astype(f64))
            q = np.where(valid, np.clip(q, 0, qmax), 0)
            gmn = np.where(live, gmn, f32(0)).astype(f32)
        else:
            sc = _one_if_zero((_max_abs(grp, valid) / f32(mid)).astype(f32))
            q = go_round(grp.astype(f64) / sc.astype(f64)[:, None]) + mid
            q = np.where(valid, np.clip(q, 0, qmax), mid)
            gmn = np.zeros(ng, f32)
        sc = np.where(live, sc, f32(1)).astype(f32)
        q = np.where(live[:, None], q, 0).astype(np.uint32)
        sc_sb, mn_sb = sc.reshape(nsb, 16), gmn.reshape(nsb, 16)
        d = _one_if_zero(sc_sb.max(axis=1).astype(f32))
        dmin = np.abs(mn_sb).max(axis=1).astype(f32)
        dmin = _one_if_zero(dmin) if has_dmin else np.zeros(nsb, f32)
        su = np.clip(go_round(sc_sb.astype(f64) / d.astype(f64)[:, None] * 255), 0, 255).astype(np.uint8)
        parts = [_f32_bytes(d), _f32_bytes(dmin), su]
        if has_dmin:
            mu = np.clip(go_round(mn_sb.astype(f64) / dmin.astype(f64)[:, None] * 127), -127, 127)
            parts.append(mu.astype(np.int8).view(np.uint8))
        parts.append(_codes_to_bytes(q, bits).reshape(nsb, 32 * bits))
        return np.concatenate(parts, axis=1).reshape(-1), e, e
    if fmt in IQ_SPEC:
        bits, group, nonlinear, mid = IQ_SPEC[fmt]
        blk, valid = _blocks(w, group)
        amax = _max_abs(blk, valid)
        qmax = (1 << bits) - 1
        if nonlinear:
            scale = _one_if_zero(amax)
            target = (blk / scale[:, None]).astype(f32)
            err = np.abs((IQ4NL[None, None, :] - target[:, :, None]).astype(f32))
            q = np.where(valid, np.argmin(err, axis=2), 0)
        elif bits == 1:
            scale = _one_if_zero(amax)
            q = np.where(valid & (blk >= 0), 1, 0)
        else:
            denom = f32(max(f32(qmax) - f32(mid), f32(1)))
            scale = _one_if_zero((amax / denom).astype(f32))
            q = go_round(blk.astype(f64) / scale.astype(f64)[:, None] + f64(f32(mid)))
            q = np.where(valid, np.clip(q, 0, qmax), 0)
        return _codes_to_bytes(q.astype(np.uint32), bits), scale, e
    if fmt == "TernaryPacked":
        blk, valid = _blocks(w, 16)
        scale = _one_if_zero(_abs_mean(blk, valid))
        q = np.clip(go_round((blk / scale[:, None]).astype(f32).astype(f64)), -1, 1) + 1
        q = np.where(valid, q, 1).astype(np.uint32)
        return _codes_to_bytes(q, 2), scale, e
    if fmt == "BinaryPacked" and block_weights == 128:
        blk, valid = _blocks(w, 128)  # cols % 128 == 0 makes flat groups row-aligned
        sg = _abs_mean(blk, valid)
        v = (-(-sg)).astype(f32)
        v = np.where(v == 0, ((f32(2) * sg) * f32(0.5)).astype(f32), v)
        v = _one_if_zero(v)
        return _codes_to_bytes((blk >= 0).astype(np.uint32), 1), v, e
    if fmt == "BinaryPacked":
        blk, valid = _blocks(w, 32)
        scale = _one_if_zero(_abs_mean(blk, valid))
        return _codes_to_bytes((valid & (blk >= 0)).astype(np.uint32), 1), scale, e
    if fmt == "AffinePacked":
        g = block_weights or 64
        blk, _ = _blocks(w, g)
        mn, mx = _min_max(blk)
        s = ((mx - mn).astype(f32) / f32(15)).astype(f32)
        bad = (s == 0) | ~np.isfinite(s)
        s = np.where(bad, f32(1), s).astype(f32)
        mn = np.where(bad, f32(0), mn).astype(f32)
        inv = (f32(1) / s).astype(f32)
        code = go_round((((blk - mn[:, None]).astype(f32)) * inv[:, None]).astype(f32).astype(f64))
        return _codes_to_bytes(np.clip(code, 0, 15).astype(np.uint32), 4), s, mn
    raise ValueError(fmt)


# ---------------------------------------------------------------- unpack
def unpack(fmt: str, rows: int, cols: int, raw, scales=None, mins=None, block_weights: int = 0):
    n = rows * cols
    raw = np.asarray(raw, np.uint8)
    if fmt in ("Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0"):
        bb = {"Q4_0": 20, "Q4_1": 24, "Q5_0": 24, "Q5_1": 28, "Q8_0": 36}[fmt]
        blk = raw.reshape(-1, bb)
        nb = blk.shape[0]
        scale = np.ascontiguousarray(blk[:, 0:4]).view(f32).reshape(nb, 1)
        if fmt == "Q4_0":
            by = blk[:, 4:].astype(np.int32)
            q = np.stack([by & 0xF, by >> 4], axis=2).reshape(nb, 32)
            q = np.where(q > 7, q - 16, q)
            out = (q.astype(f32) * scale).astype(f32)
        elif fmt == "Q4_1":
            mn = np.ascontiguousarray(blk[:, 4:8]).view(f32).reshape(nb, 1)
            by = blk[:, 8:].astype(np.int32)
            q = np.stack([by & 0xF, by >> 4], axis=2).reshape(nb, 32)
            out = (mn + (q.astype(f32) * scale).astype(f32)).astype(f32)
        elif fmt == "Q5_0":
            q = _bytes_to_codes(np.ascontiguousarray(blk[:, 4:]).reshape(-1), 5, nb * 32).reshape(nb, 32).astype(np.int32) - 16
            out = (q.astype(f32) * scale).astype(f32)
        elif fmt == "Q5_1":
            mn = np.ascontiguousarray(blk[:, 4:8]).view(f32).reshape(nb, 1)
            q = _bytes_to_codes(np.ascontiguousarray(blk[:, 8:]).reshape(-1), 5, nb * 32).reshape(nb, 32)
            out = (mn + (q.astype(f32) * scale).astype(f32)).astype(f32)
        else:
            q = np.ascontiguousarray(blk[:, 4:]).view(np.int8)
            out = (q.astype(f32) * scale).astype(f32)
        return out.reshape(-1)[:n]
    if fmt in K_SPEC:
        bits, has_dmin, qmax, mid = K_SPEC[fmt]
        sbb = 24 + (16 if has_dmin else 0) + 32 * bits
        sb = raw.reshape(-1, sbb)
        nsb = sb.shape[0]
        d = np.ascontiguousarray(sb[:, 0:4]).view(f32).reshape(nsb, 1)
        dmin = np.ascontiguousarray(sb[:, 4:8]).view(f32).reshape(nsb, 1)
        su = sb[:, 8:24].astype(f32)
        sc = ((d * su).astype(f32) / f32(255)).astype(f32)
        sc = np.where(sc == 0, (d / f32(255)).astype(f32), sc).astype(f32)
        qo = 40 if has_dmin else 24
        q = _bytes_to_codes(np.ascontiguousarray(sb[:, qo:]).reshape(-1), bits, nsb * 256).reshape(nsb, 16, 16)
        if has_dmin:
            mu = np.ascontiguousarray(sb[:, 24:40]).view(np.int8).astype(f32)
            mn = ((dmin * mu).astype(f32) / f32(127)).astype(f32)
            out = (mn[:, :, None] + (q.astype(f32) * sc[:, :, None]).astype(f32)).astype(f32)
        else:
            out = (sc[:, :, None] * (q.astype(np.int32) - mid).astype(f32)).astype(f32)
        return out.reshape(-1)[:n]
    if fmt in IQ_SPEC:
        bits, group, nonlinear, mid = IQ_SPEC[fmt]
        scales = np.asarray(scales, f32)
        q = _bytes_to_codes(raw, bits, scales.size * group).reshape(-1, group)
        sc = scales.reshape(-1, 1)
        if nonlinear:
            out = (sc * IQ4NL[q & 15]).astype(f32)
        elif bits == 1:
            out = np.where((q & 1) != 0, sc, -sc).astype(f32)
        else:
            out = (sc * (q.astype(f32) - f32(mid)).astype(f32)).astype(f32)
        return out.reshape(-1)[:n]
    if fmt == "TernaryPacked":
        sc = np.asarray(scales, f32).reshape(-1, 1)
        q = _bytes_to_codes(raw, 2, sc.size * 16).reshape(-1, 16)
        out = np.where(q == 0, -sc, np.where(q == 2, sc, f32(0))).astype(f32)
        return out.reshape(-1)[:n]
    if fmt == "BinaryPacked":
        g = 128 if block_weights == 128 else 32
        sc = np.asarray(scales, f32).reshape(-1, 1)
        q = _bytes_to_codes(raw, 1, sc.size * g).reshape(-1, g)
        return np.where(q != 0, sc, -sc).astype(f32).reshape(-1)[:n]
    if fmt == "AffinePacked":
        g = block_weights or 64
        sc = np.asarray(scales, f32).reshape(-1, 1)
        be = np.asarray(mins, f32).reshape(-1, 1)
        q = _bytes_to_codes(raw, 4, sc.size * g).reshape(-1, g)
        return ((sc * q.astype(f32)).astype(f32) + be).astype(f32).reshape(-1)[:n]
    raise ValueError(fmt)


def f16_trunc(w):
    """core.Float32ToFloat16: truncating, flush-to-zero, overflow to inf."""
    b = np.asarray(w, f32).view(np.uint32)
    sign = ((b >> 16) & 0x8000).astype(np.uint32)
    expo = ((b >> 23) & 0xFF).astype(np.int64) - 127 + 15
    mant = b & 0x7FFFFF
    body = (np.clip(expo, 0, 31).astype(np.uint32) << 10) | (mant >> 13)
    out = np.where(expo <= 0, sign, np.where(expo >= 31, sign | 0x7C00, sign | body))
    return out.astype(np.uint16)


def bf16_trunc(w):
    return (np.asarray(w, f32).view(np.uint32) >> 16).astype(np.uint16)
