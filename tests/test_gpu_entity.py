"""`.entity` ingestion straight to the device cache and quant.DecodeRow: a container written in the reference's
layout (magic, version, header JSON, payload of packed wire forms) is opened, each packed blob goes from the mapped
file into the cache without a host unpack, and the resident weights and GEMV match the oracle's."""
import numpy as np
import pytest
import torch

import oracle as O
from conftest import CASES, case_id, case_ok, to_product_blob

pytestmark = pytest.mark.gpu


def _entity(wv, tmp_path, cases, rows, cols):
    ent = wv.entity
    payload, blobs, obs = b"", [], {}
    for n, c in enumerate(cases):
        f, bw, dt = c
        w = np.random.default_rng(100 + n).normal(0, 0.02, rows * cols).astype(np.float32)
        ob = O.pack(f, w, rows, cols, bw, dt)
        name = f"transformer.layers.{n}.{case_id(c)}.weight"
        if f == "none":
            wire = ob.raw.tobytes()
            blobs.append(ent.WeightBlob(name, len(payload), len(wire), {1: "FLOAT32", 2: "FLOAT16", 3: "BFLOAT16"}[dt], "none", rows, cols, Native=True))
        else:
            wire = O.wire_encode(ob).tobytes()
            assert wire == ent.EncodePackedBlob(to_product_blob(wv, ob))
            blobs.append(ent.WeightBlob(name, len(payload), len(wire), "PACKED", O.FORMATS[ob.format], rows, cols))
        payload += wire
        obs[name] = ob
    tok = b'{"model": {}}'
    blobs.append(ent.WeightBlob(ent.TokenizerBlobPath, len(payload), len(tok), "JSON", "none"))
    payload += tok
    path = str(tmp_path / "m.entity")
    ent.WriteTransformerFile(path, {"architecture": "llama", "hidden_size": cols, "vocab_size": rows}, blobs, payload)
    return path, obs


def test_entity_blobs_reach_the_device_as_written(wv, tmp_path):
    rows, cols = 96, 512
    cases = [c for c in CASES if case_ok(c, rows, cols)]
    path, obs = _entity(wv, tmp_path, cases, rows, cols)
    L = wv._lib.lib()
    x = np.random.default_rng(7).normal(0, 1, cols).astype(np.float32)
    with wv.entity.Open(path) as ef:
        hdr = ef.Header()
        assert hdr.FormatVersion == 1 and hdr.Transformer["architecture"] == "llama" and len(hdr.Blobs) == len(cases) + 1
        assert ef.LoadBlobBytes(wv.entity.TokenizerBlobPath) == b'{"model": {}}'
        for n, (name, ob) in enumerate(obs.items()):
            key = 0xE000 + n
            if ob.format == 0:
                assert ef.WarmNumericBlob(name, key) == ob.raw.size
                with pytest.raises(ValueError):
                    ef.WarmQuantBlob(name, key + 0x100)
            else:
                assert ef.WarmQuantBlob(name, key) == ob.packed_bytes
                hb = ef.LoadQuantBlob(name)       # the host-side Blob carries the same arrays
                assert hb.Raw.tobytes() == ob.raw.tobytes() and hb.Scales.tobytes() == ob.scales.tobytes()
            out = np.empty(rows * cols, np.float32)
            wv._lib.check(L.wv_unpack(key, out.ctypes.data))
            assert out.tobytes() == O.unpack(ob).tobytes(), name
            y = np.empty(rows, np.float32)
            wv._lib.check(L.wv_matvec(key, x.ctypes.data, y.ctypes.data, 1, cols, rows))
            ref = O.matvec_simd(ob, x)
            bound = O.sum_abs_wx(ob, x)
            assert np.all(np.abs(y.astype(np.float64) - ref) <= 1e-3 * bound), name
            wv._lib.check(L.wv_blob_evict(key))


def test_entity_header_errors(wv, tmp_path):
    p = tmp_path / "bad.entity"
    p.write_bytes(b"ENTITX\0\0" + bytes(12))
    with pytest.raises(ValueError, match="magic"):
        wv.entity.Open(str(p))
    p.write_bytes(b"ENTITY\0\0" + (2).to_bytes(2, "little") + bytes(10))
    with pytest.raises(ValueError, match="version"):
        wv.entity.Open(str(p))
    p.write_bytes(b"ENTITY\0\0" + (1).to_bytes(2, "little") + bytes(2) + (5).to_bytes(8, "little") + b"{]]]]")
    with pytest.raises(ValueError, match="JSON"):
        wv.entity.Open(str(p))


@pytest.mark.parametrize("case", CASES, ids=case_id)
def test_decode_row_matches_unpack(wv, case):
    """quant.DecodeRow on the device: every row equals the oracle's DecodeRow restatement and its Unpack row,
    at a shape whose rows do not start on block boundaries where the layout allows it."""
    f, bw, dt = case
    rows, cols = (12, 256) if (f == "AffinePacked" or bw == 128) else (12, 200)
    w = np.random.default_rng(5).normal(0, 0.02, rows * cols).astype(np.float32)
    ob = O.pack(f, w, rows, cols, bw, dt)
    full = O.unpack(ob).reshape(rows, cols)
    blob = to_product_blob(wv, ob)
    L = wv._lib.lib()
    key = wv.quant.EnsureResident(blob)
    for r in (0, 1, 5, rows - 1):
        got = np.empty(cols, np.float32)
        wv._lib.check(L.wv_decode_row(key, r, got.ctypes.data, cols))
        assert got.tobytes() == full[r].tobytes()
        if f != "none":
            assert O.decode_row(ob, r).tobytes() == full[r].tobytes()
            dst = np.zeros(cols + 3, np.float32)
            wv.quant.DecodeRow(blob, r, dst)
            assert dst[:cols].tobytes() == full[r].tobytes() and not dst[cols:].any()
    d = torch.zeros(cols, device="cuda")
    wv._lib.check(L.wv_decode_row_dev(key, 2, d.data_ptr(), None))
    torch.cuda.synchronize()
    assert d.cpu().numpy().tobytes() == full[2].tobytes()
    assert L.wv_decode_row(key, rows, got.ctypes.data, cols) == wv._lib.WV_ESHAPE
    assert L.wv_decode_row(key, 0, got.ctypes.data, cols - 1) == wv._lib.WV_ESHAPE
    with pytest.raises(wv.WelvetError):
        wv.quant.DecodeRow(blob, -1, np.zeros(cols, np.float32))
    if f == "none":
        with pytest.raises(wv.WelvetError, match="FormatNone"):
            wv.quant.DecodeRow(blob, 0, np.zeros(cols, np.float32))
