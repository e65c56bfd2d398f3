"""ctypes front end of the CPU oracle (welvet_oracle.c).

TEST INFRASTRUCTURE ONLY: the checker for the CUDA path. Only the test-suite, the smoke
check and the benchmark's CPU-baseline legs may import this package; the product package
never does.

The blob container mirrors quant.Blob of the reference (quant/format.go:110-131):
format, rows, cols, Raw bytes, Scales, Mins, BlockWeights — plus the FormatNone dtype.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "welvet_oracle.c")
_SO = os.path.join(_HERE, "libwelvet_oracle.so")

# quant.Format (quant/format.go:9-39)
FORMATS = [
    "none", "Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1",
    "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K",
    "IQ1_S", "IQ2_XXS", "IQ2_XS", "IQ3_XXS", "IQ3_S", "IQ4_NL", "IQ4_XS",
    "TernaryPacked", "BinaryPacked", "AffinePacked",
]
FMT = {name: i for i, name in enumerate(FORMATS)}
DT_F32, DT_F16, DT_BF16 = 1, 2, 3  # core.DType (core/dtype.go:15-17)


def build(force: bool = False) -> str:
    """Compile the C restatement with the float semantics it depends on."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared",
               "-o", _SO, _SRC, "-lm", "-lpthread"]
        subprocess.run(cmd, check=True)
    return _SO


class _CBlob(C.Structure):
    _fields_ = [
        ("format", C.c_int32), ("dtype", C.c_int32), ("rows", C.c_int32), ("cols", C.c_int32),
        ("block_weights", C.c_int32), ("_pad", C.c_int32),
        ("raw", C.c_void_p), ("nraw", C.c_uint64),
        ("scales", C.c_void_p), ("ns", C.c_uint64),
        ("mins", C.c_void_p), ("nm", C.c_uint64),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.wvo_simd_prepare.restype = C.c_void_p
        _lib.wvo_simd_prepare.argtypes = [C.c_void_p]
        _lib.wvo_simd_matvec.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        _lib.wvo_simd_free.argtypes = [C.c_void_p]
        _lib.wvo_wire_size.restype = C.c_uint64
    return _lib


@dataclass
class Blob:
    """quant.Blob of the reference, with numpy arrays for Raw / Scales / Mins."""
    format: int
    rows: int
    cols: int
    raw: np.ndarray
    scales: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))
    mins: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))
    block_weights: int = 0
    dtype: int = DT_F32

    @property
    def packed_bytes(self) -> int:
        """len(Raw) + 4 len(Scales) + 4 len(Mins): the bytes a GEMV must stream."""
        return int(self.raw.nbytes + self.scales.nbytes + self.mins.nbytes)

    def _c(self) -> _CBlob:
        self.raw = np.ascontiguousarray(self.raw, np.uint8)
        self.scales = np.ascontiguousarray(self.scales, np.float32)
        self.mins = np.ascontiguousarray(self.mins, np.float32)
        return _CBlob(self.format, self.dtype, self.rows, self.cols, self.block_weights, 0,
                      self.raw.ctypes.data, self.raw.size,
                      self.scales.ctypes.data, self.scales.size,
                      self.mins.ctypes.data, self.mins.size)


def _fmt(f) -> int:
    return FMT[f] if isinstance(f, str) else int(f)


def sizes(fmt, rows, cols, block_weights=0, dtype=DT_F32):
    nraw, ns, nm = C.c_uint64(), C.c_uint64(), C.c_uint64()
    rc = lib().wvo_sizes(_fmt(fmt), dtype, block_weights, rows, cols, C.byref(nraw), C.byref(ns), C.byref(nm))
    if rc:
        raise ValueError(f"wvo_sizes({fmt},{rows}x{cols},bw={block_weights}) -> {rc}")
    return nraw.value, ns.value, nm.value


def pack(fmt, w: np.ndarray, rows: int, cols: int, block_weights: int = 0, dtype: int = DT_F32) -> Blob:
    """quant.Pack (quant/pack.go:4-31); FormatNone encodes the native dtype; BinaryPacked
    with block_weights=128 uses the harness-defined g128 packer."""
    f = _fmt(fmt)
    w = np.ascontiguousarray(w, np.float32).reshape(-1)
    assert w.size >= rows * cols
    nraw, ns, nm = sizes(f, rows, cols, block_weights, dtype)
    b = Blob(f, rows, cols, np.zeros(nraw, np.uint8), np.zeros(ns, np.float32), np.zeros(nm, np.float32),
             block_weights, dtype)
    cb = b._c()
    rc = lib().wvo_pack(w.ctypes.data_as(C.c_void_p), C.byref(cb))
    if rc:
        raise ValueError(f"wvo_pack -> {rc}")
    b.block_weights = cb.block_weights
    return b


def unpack(b: Blob) -> np.ndarray:
    """quant.Unpack (quant/unpack.go:4-34): the bit-exact dequantised weights."""
    out = np.zeros(b.rows * b.cols, np.float32)
    cb = b._c()
    rc = lib().wvo_unpack(C.byref(cb), out.ctypes.data_as(C.c_void_p))
    if rc:
        raise ValueError(f"wvo_unpack -> {rc}")
    return out


def matvec(b: Blob, x: np.ndarray) -> np.ndarray:
    """quant.MatVec (f32, flat order); FormatNone follows weights.matVecNativeF64."""
    x = np.ascontiguousarray(x, np.float32)
    assert x.size >= b.cols
    y = np.zeros(b.rows, np.float32)
    cb = b._c()
    rc = lib().wvo_matvec(C.byref(cb), x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p))
    if rc:
        raise ValueError(f"wvo_matvec -> {rc}")
    return y


def matvec_simd(b: Blob, x: np.ndarray, threads: int = 1) -> np.ndarray:
    """dense.MatVecPackedBlob / ForwardSIMD arithmetic (f64 accumulation)."""
    x = np.ascontiguousarray(x, np.float32)
    y = np.zeros(b.rows, np.float32)
    cb = b._c()
    rc = lib().wvo_matvec_simd(C.byref(cb), x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), threads)
    if rc:
        raise ValueError(f"wvo_matvec_simd -> {rc}")
    return y


def sum_abs_wx(b: Blob, x: np.ndarray) -> np.ndarray:
    """Per row sum_j |w_rj x_j| in f64 (the tolerance denominator)."""
    x = np.ascontiguousarray(x, np.float32)
    out = np.zeros(b.rows, np.float64)
    cb = b._c()
    rc = lib().wvo_sum_abs_wx(C.byref(cb), x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p))
    if rc:
        raise ValueError(f"wvo_sum_abs_wx -> {rc}")
    return out


class SimdCache:
    """Once-built SIMD views (Ensure*SIMDCache); build time is excluded from timing as in
    the reference, matvec() is the timed call."""

    def __init__(self, b: Blob):
        self._blob = b
        self._cb = b._c()
        self._h = lib().wvo_simd_prepare(C.addressof(self._cb))
        if not self._h:
            raise ValueError("wvo_simd_prepare failed")

    def matvec(self, x: np.ndarray, y: np.ndarray, threads: int = 0) -> int:
        return lib().wvo_simd_matvec(self._h, x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), threads)

    def close(self):
        if self._h:
            lib().wvo_simd_free(self._h)
            self._h = None

    def __del__(self):
        self.close()


def wire_encode(b: Blob) -> np.ndarray:
    """weights.EncodePackedWire / EncodeBlobWire (weights/packed_wire.go:13-52)."""
    cb = b._c()
    n = lib().wvo_wire_size(C.byref(cb))
    out = np.zeros(n, np.uint8)
    lib().wvo_wire_encode(C.byref(cb), out.ctypes.data_as(C.c_void_p))
    return out


def wire_decode(fmt, rows, cols, wire: np.ndarray, dtype: int = DT_F32) -> Blob:
    """weights.DecodePackedWire (weights/packed_wire.go:55-110)."""
    f = _fmt(fmt)
    wire = np.ascontiguousarray(wire, np.uint8)
    v = [C.c_uint64() for _ in range(6)]
    bw = C.c_int()
    rc = lib().wvo_wire_decode(f, rows, cols, wire.ctypes.data_as(C.c_void_p), C.c_uint64(wire.size),
                               *[C.byref(t) for t in v], C.byref(bw))
    if rc:
        raise ValueError(f"wvo_wire_decode -> {rc}")
    ns, nm, nr, os_, om, orr = [t.value for t in v]
    scales = wire[os_:os_ + 4 * ns].copy().view(np.float32)
    mins = wire[om:om + 4 * nm].copy().view(np.float32)
    raw = wire[orr:orr + nr].copy()
    return Blob(f, rows, cols, raw, scales, mins, bw.value, dtype)


def argmax(logits: np.ndarray) -> int:
    """sampling.ArgMax (model/sampling/argmax.go:4-18)."""
    v = np.ascontiguousarray(logits, np.float32).reshape(-1)
    return int(lib().wvo_argmax(v.ctypes.data_as(C.c_void_p), C.c_int64(v.size)))


def topk_sample(logits: np.ndarray, top_k: int, temperature: float, deterministic: bool, u: float) -> int:
    """sampling.SampleTopK (model/sampling/topk.go:11-50); u stands for the reference's rand.Float64()."""
    v = np.ascontiguousarray(logits, np.float32).reshape(-1)
    f = lib().wvo_topk_sample
    f.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_int, C.c_double]
    return int(f(v.ctypes.data_as(C.c_void_p), v.size, int(top_k), float(temperature), 1 if deterministic else 0, float(u)))


def decode_row(b: Blob, row: int) -> np.ndarray:
    """quant.DecodeRow (quant/decode_row.go:7-38)."""
    out = np.zeros(b.cols, np.float32)
    cb = b._c()
    f = lib().wvo_decode_row
    f.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int64]
    rc = f(C.byref(cb), int(row), out.ctypes.data_as(C.c_void_p), out.size)
    if rc:
        raise ValueError(f"wvo_decode_row -> {rc}")
    return out


# core.ActivationType (core/layer.go:91-98)
ACTIVATIONS = {"Linear": -1, "ReLU": 0, "SiLU": 1, "GELU": 2, "Tanh": 3, "Sigmoid": 4, "LeakyReLU": 5, "ReLU2": 6}


def activate(v: np.ndarray, act: int) -> np.ndarray:
    """core.Activate (core/activate.go:6-38) element by element in f64; unknown values of `act`
    return the input unchanged, as the reference's default arm does."""
    L = lib()
    L.wvo_activate.restype = C.c_double
    L.wvo_activate.argtypes = [C.c_double, C.c_int, C.POINTER(C.c_int)]
    a = np.asarray(v, np.float64).reshape(-1)
    return np.array([L.wvo_activate(float(t), int(act), None) for t in a], np.float64).reshape(np.shape(v))


def rmsnorm(x: np.ndarray, gamma: np.ndarray, eps: float = 1e-5) -> np.ndarray:
    """rmsnorm.Forward post output for float32 rows (layers/rmsnorm/cpu.go:32-90)."""
    x = np.ascontiguousarray(x, np.float32)
    g = np.ascontiguousarray(gamma, np.float32)
    x2 = x.reshape(-1, g.size)
    y = np.zeros_like(x2)
    lib().wvo_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_double]
    lib().wvo_rmsnorm(x2.ctypes.data, g.ctypes.data, None, y.ctypes.data, x2.shape[0], g.size, float(eps))
    return y.reshape(x.shape)


def rope(vec: np.ndarray, pos: int, num_heads: int, head_dim: int, theta: float = 10000.0) -> np.ndarray:
    """applyRoPE (layers/mha/rope.go:6-21) on a float64 copy of vec."""
    v = np.array(vec, np.float64).reshape(-1).copy()
    lib().wvo_rope.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_double]
    lib().wvo_rope(v.ctypes.data, int(pos), int(num_heads), int(head_dim), float(theta))
    return v


def attn_decode(q, cache_k, cache_v, num_heads, num_kv_heads, head_dim, kv_len, msl, scale=None) -> np.ndarray:
    """attnForward for one query token under the causal mask (layers/mha/attn.go:15-120), float64."""
    q = np.ascontiguousarray(q, np.float64).reshape(-1)
    ck = np.ascontiguousarray(cache_k, np.float64)
    cv = np.ascontiguousarray(cache_v, np.float64)
    out = np.zeros(num_heads * head_dim, np.float64)
    if scale is None:
        scale = 1.0 / np.sqrt(head_dim)
    lib().wvo_attn_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double]
    lib().wvo_attn_decode(q.ctypes.data, ck.ctypes.data, cv.ctypes.data, out.ctypes.data, num_heads, num_kv_heads, head_dim, kv_len, msl, float(scale))
    return out


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """simd.SiluMulF32 (simd/silu.go:7-27)."""
    g = np.ascontiguousarray(gate, np.float32).reshape(-1)
    u = np.ascontiguousarray(up, np.float32).reshape(-1)
    out = np.zeros_like(g)
    lib().wvo_silu_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    lib().wvo_silu_mul(g.ctypes.data, u.ctypes.data, out.ctypes.data, g.size)
    return out
