"""Host-side mirror of the reference's `.entity` checkpoint reader for the weight payloads the Dense path
consumes (model/entity/doc.go:13-22, file.go:16-27,119-263, packed.go:12-76, write.go:45-83).

Container: 8-byte magic "ENTITY\\0\\0" | u16 version (1) | u16 flags | u64 header length | header JSON | payload.
The JSON's `blobs` array indexes the payload: {path, offset, length, dtype, format, rows, cols, shape, scale,
native}; a packed blob's bytes are the packed wire form (u32 ns | u32 nm | u32 nr | scales | mins | raw).

WarmQuantBlob hands those bytes to the device cache as they lie in the file (wv_blob_upload_wire parses the
12-byte prefix and re-lays the planes on the device): nothing is unpacked on the host.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from . import _lib, quant, weights
from ._lib import WelvetError, check, lib

Magic = b"ENTITY\x00\x00"
FormatVersion = 1
headerMaxSize = 256 << 20
TokenizerBlobPath = "transformer.tokenizer.json"
_FIXED = 20


@dataclass
class WeightBlob:
    """One payload in the blob section (model/entity/file.go:16-27)."""
    Path: str
    Offset: int
    Length: int
    DType: str = ""
    Format: str = ""
    Rows: int = 0
    Cols: int = 0
    Shape: list = field(default_factory=list)
    Scale: float = 0.0
    Native: bool = False

    def to_json(self) -> dict:
        d = {"path": self.Path, "offset": self.Offset, "length": self.Length, "dtype": self.DType, "format": self.Format}
        if self.Rows:
            d["rows"] = self.Rows
        if self.Cols:
            d["cols"] = self.Cols
        if self.Shape:
            d["shape"] = list(self.Shape)
        if self.Scale:
            d["scale"] = self.Scale
        d["native"] = self.Native
        return d


@dataclass
class Header:
    FormatVersion: int
    Flags: int
    Transformer: Optional[dict]
    Blobs: list
    DataOffset: int
    Status: str = ""
    Engine: str = ""


_DTYPES = {"FLOAT32": quant.DTypeFloat32, "F32": quant.DTypeFloat32, "": quant.DTypeFloat32,
           "FLOAT16": quant.DTypeFloat16, "F16": quant.DTypeFloat16, "FP16": quant.DTypeFloat16,
           "BFLOAT16": quant.DTypeBFloat16, "BF16": quant.DTypeBFloat16}


class File:
    """Random-access `.entity` reader (model/entity/file.go:113-263); the payload is memory-mapped."""

    def __init__(self, path: str):
        self._f = open(path, "rb")
        try:
            self._read_header()
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except Exception:
            self._f.close()
            raise

    def _read_header(self) -> None:
        fixed = self._f.read(_FIXED)
        if len(fixed) < _FIXED:
            raise ValueError("entity fixed header: short read")
        if fixed[:8] != Magic:
            raise ValueError(f"invalid entity magic: {fixed[:8]!r} (want ENTITY)")
        version, flags, hlen = struct.unpack_from("<HHQ", fixed, 8)
        if version != FormatVersion:
            raise ValueError(f"unsupported entity version: {version}")
        if hlen > headerMaxSize:
            raise ValueError(f"entity header size unreasonable: {hlen}")
        raw = self._f.read(hlen)
        if len(raw) < hlen:
            raise ValueError("entity header JSON: short read")
        try:
            doc = json.loads(raw)
        except json.JSONDecodeError as e:
            raise ValueError(f"entity header JSON: {e}") from None
        blobs = [WeightBlob(b.get("path", ""), int(b.get("offset", 0)), int(b.get("length", 0)), b.get("dtype", ""),
                            b.get("format", ""), int(b.get("rows", 0)), int(b.get("cols", 0)), list(b.get("shape") or []),
                            float(b.get("scale", 0.0)), bool(b.get("native", False))) for b in doc.get("blobs") or []]
        self.hdr = Header(version, flags, doc.get("transformer"), blobs, _FIXED + hlen, doc.get("status", ""), doc.get("engine", ""))

    def Close(self) -> None:
        if self._f is not None:
            self._map.close()
            self._f.close()
            self._f = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.Close()

    def Header(self) -> Header:
        return self.hdr

    def findBlob(self, path: str) -> WeightBlob:
        for b in self.hdr.Blobs:
            if b.Path == path:
                return b
        raise KeyError(f"entity blob {path!r} not found")

    def _view(self, blob: WeightBlob) -> memoryview:
        off = self.hdr.DataOffset + blob.Offset
        if off + blob.Length > len(self._map):
            raise ValueError(f"entity blob {blob.Path!r}: payload runs past the end of the file")
        return memoryview(self._map)[off:off + blob.Length]

    def LoadBlobBytes(self, path: str) -> bytes:
        return bytes(self._view(self.findBlob(path)))

    def _packed(self, path: str):
        blob = self.findBlob(path)
        fmt = quant.ParseFormatName(blob.Format)
        if fmt == quant.Format.FormatNone:
            raise ValueError(f"entity blob {path!r}: not a packed quant blob (format={blob.Format!r})")
        if blob.Rows <= 0 or blob.Cols <= 0:
            raise ValueError(f"entity blob {path!r}: missing rows/cols")
        return blob, fmt

    def LoadQuantBlob(self, path: str) -> quant.Blob:
        """File.LoadQuantBlob + DecodePackedBlob (file.go:233-250, packed.go:37-76): a host-side Blob."""
        blob, fmt = self._packed(path)
        return weights.DecodePackedWire(fmt, blob.Rows, blob.Cols, self.LoadBlobBytes(path))

    def WarmQuantBlob(self, path: str, key: int) -> int:
        """The packed payload straight from the mapped file into the device cache under `key` (no host unpack).
        Returns the packed bytes now resident."""
        blob, fmt = self._packed(path)
        view = np.frombuffer(self._view(blob), np.uint8)
        check(lib().wv_blob_upload_wire(key, int(fmt), quant.DTypeFloat32, blob.Rows, blob.Cols, view.ctypes.data, view.size))
        return int(view.size) - 12

    def WarmNumericBlob(self, path: str, key: int, rows: int = 0, cols: int = 0) -> int:
        """A FormatNone matrix blob (FLOAT32 / FLOAT16 / BFLOAT16 elements) into the device cache as it lies in the file.
        rows / cols default to the header's; other dtypes are refused (the reference's LoadBlob widens them on the host)."""
        blob = self.findBlob(path)
        fmt = blob.Format.strip().lower()
        if fmt not in ("", "none"):
            raise ValueError(f"entity blob {path!r}: packed format {blob.Format!r} — use WarmQuantBlob")
        dt = _DTYPES.get(blob.DType.strip().upper())
        if dt is None:
            raise WelvetError(_lib.WV_EFORMAT, f"entity blob {path!r}: dtype {blob.DType!r} has no device layout")
        rows, cols = rows or blob.Rows, cols or blob.Cols
        if rows <= 0 or cols <= 0:
            raise ValueError(f"entity blob {path!r}: missing rows/cols")
        view = np.frombuffer(self._view(blob), np.uint8)
        check(lib().wv_blob_upload_wire(key, 0, dt, rows, cols, view.ctypes.data, view.size))
        return int(view.size)


def Open(path: str) -> File:
    return File(path)


def EncodePackedBlob(b: quant.Blob) -> bytes:
    """entity.EncodePackedBlob (packed.go:12-34): same bytes as weights.EncodePackedWire for a packed blob."""
    return struct.pack("<III", b.Scales.size, b.Mins.size, b.Raw.size) + b.Scales.tobytes() + b.Mins.tobytes() + b.Raw.tobytes()


def WriteTransformerFile(outPath: str, spec: Optional[dict], blobs: list, payload: bytes) -> None:
    """entity.WriteTransformerFile / writeEntityFile (write.go:13-83): magic, version, flags 0, header length, JSON, payload."""
    if spec is None:
        raise ValueError("entity.WriteTransformerFile: nil spec")
    doc = {"format_version": FormatVersion, "engine": spec.get("engine") or "welvet", "status": "packed", "transformer": spec}
    doc["blobs"] = [b.to_json() for b in blobs]
    hj = json.dumps(doc, separators=(",", ":")).encode()
    if len(hj) > headerMaxSize:
        raise ValueError(f"entity header too large: {len(hj)}")
    with open(outPath, "wb") as f:
        f.write(Magic + struct.pack("<HHQ", FormatVersion, 0, len(hj)) + hj + payload)
