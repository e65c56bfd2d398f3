"""Host-side mirror of the reference's `quant` package surface for the CUDA backend.

Format values, names and the Blob container follow quant/format.go:9-131 of the reference;
Pack / Unpack / MatVec keep the argument meaning of quant/pack.go:4, unpack.go:4 and
matvec.go:5 but run on the device through the C ABI. Arrays are numpy; a Blob's key in the
device cache is its Python identity, as the reference keys caches by *quant.Blob address
(webgpu/binary_cache.go:198), and the entry is evicted when the Blob is collected.
"""
from __future__ import annotations

import ctypes as C
import enum
import weakref
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from ._lib import WelvetError, check, lib


class Format(enum.IntEnum):
    FormatNone = 0
    FormatQ8_0 = 1
    FormatQ4_0 = 2
    FormatQ4_1 = 3
    FormatQ5_0 = 4
    FormatQ5_1 = 5
    FormatQ2_K = 6
    FormatQ3_K = 7
    FormatQ4_K = 8
    FormatQ5_K = 9
    FormatQ6_K = 10
    FormatIQ1_S = 11
    FormatIQ2_XXS = 12
    FormatIQ2_XS = 13
    FormatIQ3_XXS = 14
    FormatIQ3_S = 15
    FormatIQ4_NL = 16
    FormatIQ4_XS = 17
    FormatTernaryPacked = 18
    FormatBinaryPacked = 19
    FormatAffinePacked = 20

    def String(self) -> str:  # quant/format.go:50-97 (ENTITY header strings)
        return "none" if self == Format.FormatNone else self.name[len("Format"):]

    def IsKQuant(self) -> bool:
        return Format.FormatQ2_K <= self <= Format.FormatQ6_K


AllFormats = list(Format)


def ParseFormatName(s: str) -> Format:  # quant/format.go:134-144
    if s in ("", "none"):
        return Format.FormatNone
    for f in AllFormats:
        if f.String() == s:
            return f
    return Format.FormatNone


# core.DType values the backend accepts for FormatNone (core/dtype.go:15-17)
DTypeFloat32, DTypeFloat16, DTypeBFloat16 = 1, 2, 3
BinaryG128Group = 128
AffineG64Group = 64


@dataclass(eq=False)
class Blob:
    """quant.Blob: opaque packed weight buffer + layout metadata."""
    Format: Format
    Rows: int
    Cols: int
    Raw: np.ndarray
    Scales: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))
    Mins: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))
    BlockWeights: int = 0
    DType: int = DTypeFloat32  # FormatNone only

    def __post_init__(self):
        self.Raw = np.ascontiguousarray(self.Raw).view(np.uint8).reshape(-1)
        self.Scales = np.ascontiguousarray(self.Scales, np.float32).reshape(-1)
        self.Mins = np.ascontiguousarray(self.Mins, np.float32).reshape(-1)

    def PackedBytes(self) -> int:
        """len(Raw) + 4 len(Scales) + 4 len(Mins): the bytes one GEMV streams."""
        return int(self.Raw.nbytes + self.Scales.nbytes + self.Mins.nbytes)


def BlobKey(b: Blob) -> int:
    return id(b)


def _evict(key: int) -> None:
    try:
        if lib().wv_blob_has(key):
            lib().wv_blob_evict(key)
    except Exception:
        pass


def EnsureResident(b: Blob, rank: int = 0, world: int = 1) -> int:
    """Upload once per Blob (idempotent), like uploadAffineLocked (webgpu/affine_cache.go:111-154).
    With world > 1 only this rank's contiguous row range is kept on the device."""
    if b is None:
        raise WelvetError(_lib.WV_EARG, "nil blob")
    key = BlobKey(b)
    L = lib()
    if L.wv_blob_has(key):
        return key
    args = (key, int(b.Format), int(b.DType), b.Rows, b.Cols, b.BlockWeights,
            b.Raw.ctypes.data, b.Raw.size, b.Scales.ctypes.data if b.Scales.size else None, b.Scales.size,
            b.Mins.ctypes.data if b.Mins.size else None, b.Mins.size)
    if world > 1:
        check(L.wv_blob_upload_shard(*args, rank, world))
    else:
        check(L.wv_blob_upload(*args))
    weakref.finalize(b, _evict, key)
    return key


def Pack(format: Format, weights: np.ndarray, rows: int, cols: int, block_weights: int = 0,
         dtype: int = DTypeFloat32) -> Blob:
    """quant.Pack on the device. BinaryPacked with block_weights=128 builds the row-aligned
    g128 layout of BlobFromMLX1Bit; FormatNone encodes dtype (f32 / f16 / bf16, truncating)."""
    w = np.ascontiguousarray(weights, np.float32).reshape(-1)
    if rows <= 0 or cols <= 0 or w.size < rows * cols:
        raise WelvetError(_lib.WV_ESHAPE, f"Pack: bad shape rows={rows} cols={cols} len={w.size}")
    nraw, ns, nm = C.c_size_t(), C.c_size_t(), C.c_size_t()
    check(lib().wv_pack_sizes(int(format), dtype, block_weights, rows, cols, C.byref(nraw), C.byref(ns), C.byref(nm)))
    raw = np.zeros(nraw.value, np.uint8)
    sc = np.zeros(ns.value, np.float32)
    mn = np.zeros(nm.value, np.float32)
    check(lib().wv_pack(int(format), dtype, block_weights, w.ctypes.data, rows, cols, raw.ctypes.data,
                        sc.ctypes.data if ns.value else None, mn.ctypes.data if nm.value else None))
    f = Format(format)
    bw = {Format.FormatNone: 1, Format.FormatTernaryPacked: 16, Format.FormatBinaryPacked: 128 if block_weights == 128 else 32,
          Format.FormatAffinePacked: block_weights or AffineG64Group}.get(f, 256 if f.IsKQuant() else 32)
    return Blob(f, rows, cols, raw, sc, mn, bw, dtype)


def Unpack(b: Blob) -> np.ndarray:
    """quant.Unpack: dequantised f32 weights, bit-identical to the reference's."""
    key = EnsureResident(b)
    out = np.empty(b.Rows * b.Cols, np.float32)
    check(lib().wv_unpack(key, out.ctypes.data))
    return out


def MatVec(b: Blob, x: np.ndarray, y: np.ndarray) -> None:
    """quant.MatVec: y = W x; len(x) >= Cols and len(y) >= Rows else error (quant/helpers.go:94-103)."""
    if b is None:
        raise WelvetError(_lib.WV_EARG, "MatVec: nil blob")
    if x.size < b.Cols or y.size < b.Rows:
        raise WelvetError(_lib.WV_ESHAPE, f"MatVec: size mismatch rows={b.Rows} cols={b.Cols} len(x)={x.size} len(y)={y.size}")
    key = EnsureResident(b)
    xs = np.ascontiguousarray(x[: b.Cols], np.float32)
    ys = np.empty(b.Rows, np.float32)
    check(lib().wv_matvec(key, xs.ctypes.data, ys.ctypes.data, 1, b.Cols, b.Rows))
    y[: b.Rows] = ys


def DecodeRow(b: Blob, row: int, dst: np.ndarray) -> None:
    """quant.DecodeRow (quant/decode_row.go:7-38): one output row of a packed Blob into dst (len >= Cols)."""
    if b is None:
        raise WelvetError(_lib.WV_EFORMAT, "DecodeRow: nil blob")
    if row < 0 or row >= b.Rows or dst.size < b.Cols:
        raise WelvetError(_lib.WV_ESHAPE, f"quant: DecodeRow shape row={row} cols={b.Cols} dst={dst.size}")
    if b.Format == Format.FormatNone:
        raise WelvetError(_lib.WV_EFORMAT, "quant: DecodeRow FormatNone — use weights.DecodeRow")
    key = EnsureResident(b)
    out = np.empty(b.Cols, np.float32)
    check(lib().wv_decode_row(key, row, out.ctypes.data, out.size))
    dst[: b.Cols] = out
