"""CPU tests of the boundary and the host-side mirror: the shared library loads and exports
every symbol the header declares, status codes without a device, size formulas against the
oracle, shard ranges, the wire codec of the host mirror, and a two-rank gloo run of the
row-shard bookkeeping."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import oracle as O
from conftest import CASES, case_id, case_ok, make_w, ROOT


def _lib():
    from welvet_b200 import _lib
    return _lib


def test_library_exports_every_declared_symbol():
    L = _lib().lib()
    header = open(os.path.join(ROOT, "include", "welvet_cuda.h")).read()
    declared = set(re.findall(r"\b(wv_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib().SYMBOLS), declared ^ set(_lib().SYMBOLS)
    for s in declared:
        assert hasattr(L, s), s


def test_product_library_has_no_development_hooks():
    """The product library exports the declared ABI and none of the tuning hooks; the variant the tests load
    (built with -DWV_DEV_HOOKS) exports both."""
    m = _lib()
    here = os.path.join(ROOT, "welvet_b200")
    prod = C.CDLL(os.path.join(here, "libwelvet_cuda.so"))
    for s in m.SYMBOLS:
        assert hasattr(prod, s), s
    for s in m.DEV_HOOKS:
        assert not hasattr(prod, s), s
    dev_path = os.path.join(here, "libwelvet_cuda_dev.so")
    if os.path.exists(dev_path):
        dev = C.CDLL(dev_path)
        for s in m.SYMBOLS + m.DEV_HOOKS:
            assert hasattr(dev, s), s


def test_status_codes_without_a_device():
    m = _lib()
    L = m.lib()
    if L.wv_device_count() > 0:
        pytest.skip("a device is present")
    assert L.wv_available() == 0
    assert L.wv_init(0) == m.WV_EINIT and b"no CUDA device" in L.wv_last_error()
    x = np.zeros(8, np.float32)
    assert L.wv_matvec(1, x.ctypes.data, x.ctypes.data, 1, 8, 8) == m.WV_EINIT  # no CPU fallback
    assert L.wv_blob_has(1) == 0 and L.wv_cache_bytes() == 0
    # every compute entry fails the same way: nothing runs on the host
    keys, outs, ptrs = (C.c_uint64 * 1)(1), (C.c_int * 1)(8), (C.c_void_p * 1)(x.ctypes.data)
    idx, p, h = C.c_int(), C.c_void_p(), C.create_string_buffer(64)
    assert L.wv_matvec_dev(1, x.ctypes.data, x.ctypes.data, 1, 8, 8, None) == m.WV_EINIT
    assert L.wv_matvec_dev_static(1, x.ctypes.data, x.ctypes.data, 8, 8, None) == m.WV_EINIT
    assert L.wv_matvec_dev_multi(keys, 1, x.ctypes.data, ptrs, 1, 8, outs, None) == m.WV_EINIT
    assert L.wv_matvec_dev_gather(1, x.ctypes.data, ptrs, 1, 0, 0, 8, 8, None) == m.WV_EINIT
    assert L.wv_argmax(x.ctypes.data, 8, C.byref(idx), None) == m.WV_EINIT
    assert L.wv_gather_alloc(64, C.byref(p), h) == m.WV_EINIT
    assert L.wv_unpack(1, x.ctypes.data) == m.WV_EINIT
    assert L.wv_pack(2, 1, 0, x.ctypes.data, 1, 8, x.ctypes.data, None, None) == m.WV_EINIT


@pytest.mark.parametrize("case", CASES, ids=case_id)
def test_pack_sizes_match_oracle(case):
    f, bw, dt = case
    L = _lib().lib()
    for rows, cols in ((8, 256), (3, 100), (5, 4096), (1, 31)):
        if not case_ok(case, rows, cols):
            continue
        a, b, c = C.c_size_t(), C.c_size_t(), C.c_size_t()
        assert L.wv_pack_sizes(O.FMT[f], dt, bw, rows, cols, C.byref(a), C.byref(b), C.byref(c)) == 0
        assert (a.value, b.value, c.value) == O.sizes(f, rows, cols, bw, dt)


def test_pack_sizes_errors_and_shard_range():
    m = _lib()
    L = m.lib()
    a = C.c_size_t()
    assert L.wv_pack_sizes(2, 1, 0, 0, 5, C.byref(a), None, None) == m.WV_ESHAPE
    assert L.wv_pack_sizes(99, 1, 0, 4, 32, C.byref(a), None, None) == m.WV_EFORMAT
    assert L.wv_pack_sizes(0, 7, 0, 4, 32, C.byref(a), None, None) == m.WV_EFORMAT
    assert L.wv_pack_sizes(20, 1, 64, 4, 96, C.byref(a), None, None) == m.WV_ESHAPE   # affine cols % group
    assert L.wv_pack_sizes(19, 1, 128, 4, 96, C.byref(a), None, None) == m.WV_ESHAPE  # g128 cols % 128
    lo, hi = C.c_int(), C.c_int()
    covered = []
    for r in range(8):
        assert L.wv_shard_range(128256, r, 8, C.byref(lo), C.byref(hi)) == 0
        covered.append((lo.value, hi.value))
    assert covered[0][0] == 0 and covered[-1][1] == 128256
    assert all(covered[i][1] == covered[i + 1][0] for i in range(7)) and all(h - l == 16032 for l, h in covered)
    assert L.wv_shard_range(10, 3, 3, C.byref(lo), C.byref(hi)) == m.WV_EARG


def test_host_mirror_wire_codec_matches_oracle():
    from welvet_b200 import quant, weights
    rows, cols = 6, 256
    w, _ = make_w(2, rows, cols)
    for f, bw in (("Q4_K", 0), ("IQ3_S", 0), ("BinaryPacked", 128), ("AffinePacked", 64), ("TernaryPacked", 0)):
        ob = O.pack(f, w, rows, cols, bw)
        pb = quant.Blob(quant.Format(ob.format), rows, cols, ob.raw, ob.scales, ob.mins, ob.block_weights)
        wire = weights.EncodePackedWire(pb)
        assert wire == O.wire_encode(ob).tobytes()
        back = weights.DecodePackedWire(pb.Format, rows, cols, wire)
        assert np.array_equal(back.Raw, ob.raw) and np.array_equal(back.Scales, ob.scales) and np.array_equal(back.Mins, ob.mins)
        if f == "BinaryPacked":
            assert back.BlockWeights == 128
    with pytest.raises(Exception):
        weights.DecodePackedWire(quant.Format.FormatQ4_K, rows, cols, wire[:20])
    assert quant.ParseFormatName("Q4_K") == quant.Format.FormatQ4_K and quant.Format.FormatIQ2_XXS.String() == "IQ2_XXS"
    assert quant.ParseFormatName("") == quant.Format.FormatNone and quant.Format.FormatQ6_K.IsKQuant()


WORKER = r'''
import os, sys, ctypes as C
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["WV_ROOT"])
import oracle as O
from welvet_b200 import _lib
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
L = _lib.lib()
rows, cols = 64, 512
w = np.random.default_rng(11).normal(0, 0.02, (rows, cols)).astype(np.float32)
x = np.random.default_rng(12).normal(0, 1, cols).astype(np.float32)
lo, hi = C.c_int(), C.c_int()
assert L.wv_shard_range(rows, rank, world, C.byref(lo), C.byref(hi)) == 0
# each rank computes its slice with the oracle standing in for the device, then all-gathers
ob = O.pack("Q4_K", w[lo.value:hi.value], hi.value - lo.value, cols)
part = torch.from_numpy(O.matvec_simd(ob, x, 1))
full = torch.zeros(rows)
dist.all_gather_into_tensor(full, part)
ref = O.matvec_simd(O.pack("Q4_K", w, rows, cols), x, 1)
assert np.array_equal(full.numpy(), ref), "row shards do not reassemble"
dist.barrier()
dist.destroy_process_group()
'''


def test_row_shard_bookkeeping_two_ranks_gloo(tmp_path):
    """Sharding by contiguous row ranges + all-gather reproduces the unsharded result (flat
    block boundaries coincide with the shard boundaries)."""
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, WV_ROOT=ROOT, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29531", str(script)],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]


BLOCK_WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["WV_ROOT"])
import oracle as O
from welvet_b200.decode import BlockConfig, projection_shapes, shard_plan, vector_layout
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
cfg = BlockConfig(256, 4, 2, 64, 512, 16)
shapes, plan, lay = projection_shapes(cfg), shard_plan(cfg, rank, world), vector_layout(cfg)
rng = np.random.default_rng(21)
W = {n: rng.normal(0, 0.05, s).astype(np.float32) for n, s in shapes.items()}
ck = rng.normal(0, 1, (cfg.MaxSeqLen, 128)); cv = rng.normal(0, 1, (cfg.MaxSeqLen, 128))
x = rng.normal(0, 1, 256).astype(np.float32); g1 = rng.normal(1, 0.1, 256).astype(np.float32); g2 = rng.normal(1, 0.1, 256).astype(np.float32)
pos = 9
full = {n: O.pack("Q4_K", W[n], *shapes[n]) for n in shapes}
mine = {n: O.pack("Q4_K", W[n][plan[n][0]:plan[n][1]], plan[n][1] - plan[n][0], shapes[n][1]) for n in shapes}

def walk(mv, resid):
    """The block walk of ShardedBlockDecoder.step: mv(name, vec) is the (gathered) projection, resid adds a residual."""
    buf = np.zeros(lay["total"], np.float32)          # this rank's exchange buffer
    buf[lay["ha"]:lay["ha"] + 256] = x
    n1 = O.rmsnorm(buf[lay["ha"]:lay["ha"] + 256], g1)
    for n in ("q", "k", "v"):
        buf[lay[n]:lay[n] + shapes[n][0]] = mv(n, n1)
    k_, v_ = ck.copy(), cv.copy()
    q = O.rope(buf[lay["q"]:lay["q"] + 256], pos, 4, 64)
    k_[pos % cfg.MaxSeqLen] = O.rope(buf[lay["k"]:lay["k"] + 128], pos, 2, 64)
    v_[pos % cfg.MaxSeqLen] = buf[lay["v"]:lay["v"] + 128]
    attn = O.attn_decode(q, k_, v_, 4, 2, 64, pos + 1, cfg.MaxSeqLen).astype(np.float32)
    buf[lay["hb"]:lay["hb"] + 256] = resid("o", mv("o", attn), buf[lay["ha"]:lay["ha"] + 256])
    n2 = O.rmsnorm(buf[lay["hb"]:lay["hb"] + 256], g2)
    buf[lay["ffn"]:lay["ffn"] + 512] = O.silu_mul(mv("gate", n2), mv("up", n2))
    buf[lay["ha"]:lay["ha"] + 256] = resid("down", mv("down", buf[lay["ffn"]:lay["ffn"] + 512]), buf[lay["hb"]:lay["hb"] + 256])
    return buf[lay["ha"]:lay["ha"] + 256].copy()

def mv_full(n, vec): return O.matvec_simd(full[n], np.ascontiguousarray(vec, np.float32), 1)
def mv_sharded(n, vec):
    part = torch.from_numpy(O.matvec_simd(mine[n], np.ascontiguousarray(vec, np.float32), 1))
    out = torch.zeros(shapes[n][0])
    dist.all_gather_into_tensor(out, part)     # every rank's rows into every rank's vector
    return out.numpy()
ref = walk(mv_full, lambda n, y, r: y + r)
got = walk(mv_sharded, lambda n, y, r: y + r)      # each owner adds its own rows of the residual: same sums
assert np.array_equal(ref, got), "the sharded block walk differs from the unsharded one"
# the plan tiles every projection's rows without gaps, and the vectors of the exchange buffer do not overlap
for n, (r, _) in shapes.items():
    assert plan[n] == (r * rank // world, r * (rank + 1) // world)
offs = sorted((lay[k], k) for k in ("q", "k", "v", "ha", "hb", "ffn"))
sizes = {"q": 256, "k": 128, "v": 128, "ha": 256, "hb": 256, "ffn": 512}
for (o, k), (o2, _) in zip(offs, offs[1:] + [(lay["total"], "")]):
    assert o + sizes[k] <= o2
dist.barrier()
dist.destroy_process_group()
'''


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_block_walk_gloo(tmp_path, world):
    """The row-sharded decoder block's bookkeeping (shard plan, exchange-buffer layout, hidden state alternating between two
    vectors, residual added by the rows' owner) on two and four gloo ranks with the oracle standing in for the device: the
    sharded walk equals the unsharded one bit for bit."""
    script = tmp_path / "block_worker.py"
    script.write_text(BLOCK_WORKER)
    env = dict(os.environ, WV_ROOT=ROOT, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(29533 + world), str(script)],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]


def test_activation_values_match_the_reference_enum():
    """core.ActivationType (core/layer.go:91-98): the integers are part of the call surface, so they
    are pinned here as literals; the mirror's Activate must agree with the oracle's restatement of
    core.Activate (core/activate.go:6-38) for every one of them."""
    from welvet_b200 import dense
    want = {"ActivationLinear": -1, "ActivationReLU": 0, "ActivationSilu": 1, "ActivationGELU": 2,
            "ActivationTanh": 3, "ActivationSigmoid": 4, "ActivationLeakyReLU": 5, "ActivationReLU2": 6}
    for name, val in want.items():
        assert getattr(dense, name) == val, name
    assert sorted(O.ACTIVATIONS.values()) == sorted(want.values())
    hpp = open(os.path.join(ROOT, "welvet_b200", "host", "welvet.hpp")).read()
    body = re.search(r"enum ActivationType : int \{(.*?)\};", hpp, re.S).group(1)
    got = {k: int(v) for k, v in re.findall(r"(Activation\w+)\s*=\s*(-?\d+)", body)}
    assert got == want
    v = np.array([-30.0, -2.5, -1.0, -1e-3, 0.0, 1e-3, 0.7, 1.0, 2.5, 30.0])
    for act in want.values():
        np.testing.assert_allclose(dense.Activate(v, act), O.activate(v, act), rtol=1e-15, atol=0)
    with pytest.raises(_lib().WelvetError):
        dense.Activate(v, 7)
    np.testing.assert_array_equal(O.activate(v, 7), v)   # the reference's default arm: unchanged
