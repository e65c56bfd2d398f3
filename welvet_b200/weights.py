"""Host-side mirror of the reference's `weights` surface used by the Dense path: the Store
(weights/store.go:14-32), FromBlob (weights/from_blob.go:11-32) and the packed wire form
(weights/packed_wire.go:30-110). Byte shuffling only; all arithmetic runs on the device."""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import _lib, quant
from ._lib import WelvetError


@dataclass(eq=False)
class Store:
    """Storage truth for one weight matrix: DType + Format + packed blob (+ optional bias)."""
    DType: int
    Format: quant.Format
    Rows: int
    Cols: int
    Packed: Optional[quant.Blob] = None
    Bias: Optional[np.ndarray] = None  # float64, applied after the GEMV (dense.applyBiasAct)

    def Pack(self, format: quant.Format, block_weights: int = 0) -> None:
        """Store.Pack (weights/store.go:86-103): re-encode the current payload as `format`."""
        if self.Packed is None:
            raise WelvetError(_lib.WV_EARG, "weights: nil packed blob")
        w = quant.Unpack(self.Packed)
        self.Packed = quant.Pack(format, w, self.Rows, self.Cols, block_weights, self.DType)
        self.Format = quant.Format(format)


def New(rows: int, cols: int, data, dt: int, format: quant.Format, block_weights: int = 0) -> Store:
    """weights.New (weights/store.go:35-66): FormatNone storage in dt, then optional Pack."""
    if rows <= 0 or cols <= 0:
        raise WelvetError(_lib.WV_ESHAPE, f"weights: bad shape {rows}x{cols}")
    n = rows * cols
    src = np.zeros(n, np.float32) if data is None else np.asarray(data, np.float32).reshape(-1)
    if src.size < n:
        raise WelvetError(_lib.WV_ESHAPE, f"weights: need {n} values")
    blob = quant.Pack(format, src, rows, cols, block_weights, dt)
    return Store(dt, quant.Format(format), rows, cols, blob)


def FromBlob(b: quant.Blob) -> Store:
    if b is None:
        raise WelvetError(_lib.WV_EARG, "weights: nil blob")
    return Store(b.DType, b.Format, b.Rows, b.Cols, b)


def EncodePackedWire(b: quant.Blob) -> bytes:
    """u32 ns | u32 nm | u32 nr | scales | mins | raw, little-endian; FormatNone = raw only."""
    if b.Format == quant.Format.FormatNone:
        return b.Raw.tobytes()
    return struct.pack("<III", b.Scales.size, b.Mins.size, b.Raw.size) + b.Scales.tobytes() + b.Mins.tobytes() + b.Raw.tobytes()


def DecodePackedWire(format: quant.Format, rows: int, cols: int, wire: bytes, dtype: int = quant.DTypeFloat32) -> quant.Blob:
    """weights.DecodePackedWire: Meta / BlockWeights are not on the wire and are re-inferred
    (binary: InferBinaryBlockWeights, quant/binary_g128.go:79-94)."""
    format = quant.Format(format)
    buf = np.frombuffer(wire, np.uint8)
    if format == quant.Format.FormatNone:
        need = rows * cols * (4 if dtype == quant.DTypeFloat32 else 2)
        if buf.size < need:
            raise WelvetError(_lib.WV_ESHAPE, f"weights: FormatNone wire short {buf.size} < {need}")
        return quant.Blob(format, rows, cols, buf[:need].copy(), BlockWeights=1, DType=dtype)
    if buf.size < 12:
        raise WelvetError(_lib.WV_ESHAPE, "weights: packed wire too short")
    ns, nm, nr = struct.unpack_from("<III", wire, 0)
    need = 12 + 4 * ns + 4 * nm + nr
    if buf.size < need:
        raise WelvetError(_lib.WV_ESHAPE, f"weights: packed wire truncated (need {need}, have {buf.size})")
    scales = buf[12:12 + 4 * ns].copy().view(np.float32)
    mins = buf[12 + 4 * ns:12 + 4 * ns + 4 * nm].copy().view(np.float32)
    raw = buf[12 + 4 * ns + 4 * nm:need].copy()
    bw = 0
    if format == quant.Format.FormatBinaryPacked:
        bw = 128 if cols % 128 == 0 and ns == rows * (cols // 128) else 32
    return quant.Blob(format, rows, cols, raw, scales, mins, bw, dtype)
