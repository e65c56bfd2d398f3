"""The `.entity` container on the host: layout written and read as the reference does (magic, version, flags, header
length, JSON index, payload), packed payloads decoded into the same arrays the oracle packed. No device is touched."""
import json
import struct

import numpy as np
import pytest

import oracle as O
from welvet_b200 import entity, quant


def _blob(f, rows, cols, bw=0):
    w = np.random.default_rng(3).normal(0, 0.02, rows * cols).astype(np.float32)
    return O.pack(f, w, rows, cols, bw)


def test_entity_layout_and_packed_payloads(tmp_path):
    rows, cols = 8, 256
    obs = {"a.q4_0": _blob("Q4_0", rows, cols), "b.q4_k": _blob("Q4_K", rows, cols), "c.bin128": _blob("BinaryPacked", rows, cols, 128),
           "d.bin32": _blob("BinaryPacked", rows, cols), "e.affine": _blob("AffinePacked", rows, cols)}
    payload, blobs = b"", []
    for name, ob in obs.items():
        wire = O.wire_encode(ob).tobytes()
        blobs.append(entity.WeightBlob(name, len(payload), len(wire), "PACKED", O.FORMATS[ob.format], rows, cols))
        payload += wire
    path = str(tmp_path / "t.entity")
    entity.WriteTransformerFile(path, {"architecture": "llama", "hidden_size": cols}, blobs, payload)
    data = open(path, "rb").read()
    assert data[:8] == b"ENTITY\x00\x00" and struct.unpack_from("<HH", data, 8) == (1, 0)
    (hlen,) = struct.unpack_from("<Q", data, 12)
    doc = json.loads(data[20:20 + hlen])
    assert doc["format_version"] == 1 and doc["status"] == "packed" and doc["engine"] == "welvet"
    assert [b["path"] for b in doc["blobs"]] == list(obs) and doc["blobs"][1]["format"] == "Q4_K"
    assert data[20 + hlen:] == payload
    with entity.Open(path) as ef:
        assert ef.Header().DataOffset == 20 + hlen
        for name, ob in obs.items():
            hb = ef.LoadQuantBlob(name)
            assert (hb.Format, hb.Rows, hb.Cols) == (quant.Format(ob.format), rows, cols)
            assert hb.Raw.tobytes() == ob.raw.tobytes() and hb.Scales.tobytes() == ob.scales.tobytes() and hb.Mins.tobytes() == ob.mins.tobytes()
        assert ef.LoadQuantBlob("c.bin128").BlockWeights == 128 and ef.LoadQuantBlob("d.bin32").BlockWeights == 32
        with pytest.raises(KeyError):
            ef.LoadQuantBlob("missing")
    with pytest.raises(ValueError, match="nil spec"):
        entity.WriteTransformerFile(path, None, [], b"")


def test_entity_rejects_bad_headers(tmp_path):
    p = tmp_path / "bad.entity"
    for body, what in ((b"ENTITX\0\0" + bytes(12), "magic"), (b"ENTITY\0\0" + (2).to_bytes(2, "little") + bytes(10), "version"),
                       (b"ENTITY\0\0" + (1).to_bytes(2, "little") + bytes(2) + (5).to_bytes(8, "little") + b"{]]]]", "JSON"),
                       (b"ENTITY\0\0" + (1).to_bytes(2, "little") + bytes(2) + (300 << 20).to_bytes(8, "little"), "unreasonable"),
                       (b"ENTI", "short")):
        p.write_bytes(body)
        with pytest.raises(ValueError, match=what):
            entity.Open(str(p))
    # a numeric blob is not a packed one, and a packed blob without rows / cols is refused
    blobs = [entity.WeightBlob("n", 0, 16, "FLOAT32", "none", 2, 2), entity.WeightBlob("p", 16, 12, "PACKED", "Q4_0")]
    entity.WriteTransformerFile(str(p), {"architecture": "x"}, blobs, bytes(28))
    with entity.Open(str(p)) as ef:
        with pytest.raises(ValueError, match="not a packed"):
            ef.LoadQuantBlob("n")
        with pytest.raises(ValueError, match="rows/cols"):
            ef.LoadQuantBlob("p")
