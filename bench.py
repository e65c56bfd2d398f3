#!/usr/bin/env python
"""Benchmark of the Dense MatVec hot path (fused dequantise-and-dot GEMV).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one batch-1 GEMV for every format of the format sweep at 4096x14336 and at
14336x4096 (Llama-3-8B FFN shapes), weights N(0, 0.02^2) seed 2, activations N(0, 1) seed 1.
`value` is GB/s of packed weight bytes (len(Raw) + 4 len(Scales) + 4 len(Mins)) with everything
resident in HBM; one step streams ~1.36 GB of distinct weights, far more than L2, so no launch
reads L2-resident weights. `e2e` is the same metric through the host-pointer plugin call
(wv_matvec: host x in, host y out, copies inside the timed region).

With N > 1 (launched by torch.distributed.run) every matrix is row-sharded across the ranks and
each rank's kernels store their rows into every rank's output vectors (strong scaling).

Beside the headline: `config3` is the small-batch GEMM (M x 4096 against a 4096 x 4096 matrix in Q8_0
and Q4_K), `config4` is single-token decode of the 8B-shaped stack (32 blocks, Q4_K) on one
GPU in tokens/s, `config5` the 70B-shaped stack (80 blocks, Q4_K) and its 128256 x 8192 LM head
(Q8_0 and Q4_K) row-sharded over the N ranks, with the time the cross-rank ordering costs shown apart.

--impl reference times the CPU restatement of the reference's SIMD path (oracle/) on the host
cores over the same sweep: it is the reference arm, not the product. Both arms print the same
metric, unit and config.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "quant GEMV GB/s of packed weight bytes"
SHAPES = [(4096, 14336), (14336, 4096)]
# The format sweep: (name, quant.Format value, BlockWeights, FormatNone dtype)
SWEEP = [("Q4_0", 2, 0, 1), ("Q4_1", 3, 0, 1), ("Q5_0", 4, 0, 1), ("Q5_1", 5, 0, 1), ("Q8_0", 1, 0, 1),
         ("Q2_K", 6, 0, 1), ("Q3_K", 7, 0, 1), ("Q4_K", 8, 0, 1), ("Q5_K", 9, 0, 1), ("Q6_K", 10, 0, 1),
         ("IQ1_S", 11, 0, 1), ("IQ2_XXS", 12, 0, 1), ("IQ2_XS", 13, 0, 1), ("IQ3_XXS", 14, 0, 1), ("IQ3_S", 15, 0, 1),
         ("IQ4_NL", 16, 0, 1), ("IQ4_XS", 17, 0, 1), ("TernaryPacked", 18, 0, 1), ("BinaryPacked_g128", 19, 128, 1)]
# Measured per format but outside the timed step (named by the target, not by the sweep config).
EXTRA = [("AffinePacked_g64", 20, 64, 1), ("BinaryPacked_g32", 19, 32, 1), ("none_f16", 0, 0, 2), ("none_bf16", 0, 0, 3), ("none_f32", 0, 0, 1)]
NOMINAL_HBM_GBS = 8000.0
# DRAM bytes per launch (dram__bytes.sum.per_second x gpu__time_duration.sum) from ncu captures of single launches at
# 4096x14336, next to the algorithmic bytes of the same launches: one launch streams its blob once.
NCU_DRAM_BYTES = {"Q4_0": 36822016, "Q8_0": 66425856, "Q4_K": 38659840, "Q5_K": 46000640, "Q2_K": 23978240, "IQ4_NL": 36798464}
NCU_ALGO_BYTES = {"Q4_0": 36700160, "Q8_0": 66060288, "Q4_K": 38535168, "Q5_K": 45875200, "Q2_K": 23855104, "IQ4_NL": 36700160}
MIN_TIMED_S = 0.25   # the timed region is lengthened to at least this by replaying the step


def common_config(sweep):
    """The workload description both arms print, word for word."""
    return {"workload": "format_sweep_4096x14336+14336x4096", "formats": [f[0] for f in sweep], "batch": 1,
            "weights": "N(0,0.02^2) seed 2", "activations": "N(0,1) seed 1",
            "l2": "inputs larger than L2: one step streams 1365 MB of distinct packed weights (38 matrices, 9-66 MB each)"}


def measured_hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json, burst copy)"
    return 6650.0, "fallback (6.65 TB/s)"


class ClockSampler:
    """nvidia-smi samples during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def gen_weights(rows, cols):
    return np.random.default_rng(2).normal(0, 0.02, rows * cols).astype(np.float32)


def gen_x(cols):
    return np.random.default_rng(1).normal(0, 1, cols).astype(np.float32)


# ------------------------------------------------------------------------------ reference arm
def cpu_leg(steps, warmup, formats, shapes, threads=0):
    """Times the oracle's restatement of the reference SIMD path (dense.MatVecPackedBlob) on the host
    cores for `formats` at `shapes`; returns (GB/s of packed bytes, cores used, seconds per step, bytes)."""
    import oracle as O
    from concurrent.futures import ThreadPoolExecutor
    O.lib()
    work, total = [], 0
    for rows, cols in shapes:
        w = gen_weights(rows, cols)
        x = gen_x(cols)
        y = np.zeros(rows, np.float32)

        def prepare(spec):
            name, fmt, bw, dt = spec
            ob = O.pack(fmt, w, rows, cols, bw, dt)
            return O.SimdCache(ob), ob   # caches are built once, outside the timed loop, as in the reference
        with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:   # packing only: the timed loop below is serial
            for cache, ob in ex.map(prepare, formats):
                work.append((cache, ob, x, y))
                total += ob.packed_bytes
        del w
    cores = 1
    for _ in range(warmup):
        for c, _, x, y in work:
            cores = max(cores, c.matvec(x, y, threads))
    t0 = time.perf_counter()
    for _ in range(steps):
        for c, _, x, y in work:
            c.matvec(x, y, threads)
    dt_s = (time.perf_counter() - t0) / max(steps, 1)
    return total / dt_s / 1e9, cores, dt_s, total


def run_reference(args, rank, world):
    if rank != 0:
        return
    sweep = [f for f in SWEEP if not args.formats or f[0] in args.formats.split(",")]
    gbs, cores, sec, total = cpu_leg(args.steps, max(args.warmup, 1), sweep, SHAPES)
    desc = (f"the whole sweep per step: {len(sweep)} formats at both shapes, {total/1e6:.0f} MB packed per step, "
            f"SIMD-path caches prebuilt, {cores} host threads")
    out = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s",
           "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
           "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64 accumulate (reference SIMD path)",
           "data": "synthetic", "config": common_config(sweep),
           "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": desc},
           "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    emit(out)


# ------------------------------------------------------------------------------ product arm
_STDOUT_FD = None


def emit(obj):
    line = (json.dumps(obj) + "\n").encode()
    if _STDOUT_FD is None:
        sys.stdout.write(line.decode()); sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_STDOUT_FD, line)


def time_graph(torch, stream, graph, reps=5):
    """Best of `reps` device times of one replay of `graph` (ms), CUDA events on the launching stream."""
    best = 1e30
    with torch.cuda.stream(stream):
        graph.replay()
        stream.synchronize()
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream); graph.replay(); b.record(stream)
            stream.synchronize()
            best = min(best, a.elapsed_time(b))
    return best


def parity_sample(torch, L, _lib, O, spec, w_host, x_host, rows, cols, key, y_dev, scratch):
    """Parity beside a timed number: on three 64-row bands of the matrix the device's dequantised weights
    (wv_unpack_dev) are compared bit for bit with the oracle's Unpack, and the GEMV output that was just
    timed with the oracle's SIMD-path MatVec (max |y - y_ref| / sum|w x| over the rows). Bands are packed by
    the oracle's own packer (rows are whole blocks at these shapes, so a band packs to the bytes it has
    inside the full matrix)."""
    name, fmt, bw, dt = spec
    _lib.check(L.wv_unpack_dev(key, scratch.data_ptr(), None))
    torch.cuda.synchronize()
    y = y_dev.cpu().numpy()
    exact, worst = True, 0.0
    for r0 in (0, (rows // 2) & ~63, rows - 64):
        ob = O.pack(fmt, w_host[r0 * cols:(r0 + 64) * cols], 64, cols, bw, dt)
        want = torch.from_numpy(O.unpack(ob).view(np.int32)).cuda()
        got = scratch[r0 * cols:(r0 + 64) * cols].view(torch.int32)
        exact = exact and bool(torch.equal(want, got))
        ref = O.matvec_simd(ob, x_host, 0).astype(np.float64)
        den = O.sum_abs_wx(ob, x_host)
        worst = max(worst, float(np.max(np.abs(y[r0:r0 + 64].astype(np.float64) - ref) / np.maximum(den, 1e-30))))
    return exact, worst


MODELS = {
    # BlockConfig fields, layers, vocabulary; both decode one token at position 2048 over a cache of 2048 positions
    "8B": dict(d=4096, heads=32, kv_heads=8, head_dim=128, ffn=14336, layers=32, vocab=128256, seed=4, key=0x400000),
    "70B": dict(d=8192, heads=64, kv_heads=8, head_dim=128, ffn=28672, layers=80, vocab=128256, seed=5, key=0x500000),
}
CTX = 2048
PROJ = ("q", "k", "v", "o", "gate", "up", "down")


def _pack_rows(torch, L, _lib, key, fmt, rows, cols, r0, r1, gen):
    """N(0, 0.02^2) weights of the whole matrix from `gen` (every rank draws the same matrix), rows [r0, r1) packed on
    the device under `key`; returns the packed bytes kept."""
    w = torch.randn(rows * cols, device="cuda", generator=gen) * 0.02
    _lib.check(L.wv_pack_upload_dev(key, fmt, 1, 0, w.data_ptr() + 4 * r0 * cols, r1 - r0, cols, None))
    wb = C.c_uint64()
    _lib.check(L.wv_blob_info(key, None, None, C.byref(wb), None, None))
    del w
    return int(wb.value)


class DecodeStack:
    """A whole Llama-shaped stack for single-token decode on the device, every projection in the 4-bit k-quant and
    row-sharded over `world` ranks. Per token: embedding row, then per block Q|K|V (RMSNorm in its prologue), RoPE +
    cache write, attention over 2049 positions, O + residual, gate|up (RMSNorm in its prologue, SiLU product in its
    epilogue), down + residual; then the LM head (final RMSNorm in its prologue) and the greedy pick. All blocks have their own weights and caches."""

    def __init__(self, torch, L, _lib, name, head_formats, rank, world, exchange, layers=None, full_rows=False):
        from welvet_b200.decode import BlockConfig, ShardedBlockDecoder, projection_shapes, shard_plan, vector_layout
        from welvet_b200.dense import GatherBuffers
        m = MODELS[name]
        self.torch, self.L, self._lib, self.m, self.rank, self.world = torch, L, _lib, m, rank, world
        if full_rows:                       # the unsharded twin used to check a sharded run
            rank, world = 0, 1
        self.srank, self.sworld = rank, world
        self.layers = layers or m["layers"]
        msl = CTX + 128
        cfg = self.cfg = BlockConfig(m["d"], m["heads"], m["kv_heads"], m["head_dim"], m["ffn"], msl)
        shapes, plan, lay = projection_shapes(cfg), shard_plan(cfg, rank, world), vector_layout(cfg)
        self.lay = lay
        kd, d, vocab = cfg.NumKVHeads * cfg.HeadDim, cfg.DModel, m["vocab"]
        gen = torch.Generator(device="cuda")
        gen.manual_seed(m["seed"])
        t0 = time.perf_counter()
        key = m["key"] + (0x80000 if full_rows else 0)
        self.logits_off = lay["total"]
        self.vec = GatherBuffers(4 * (lay["total"] + ((vocab + 63) & ~63)), rank, world, exchange)
        self.flags = GatherBuffers(4 * (world + 2), rank, world, exchange) if world > 1 else None
        self.local = {"attn": torch.zeros(cfg.NumHeads * cfg.HeadDim, device="cuda")}
        self.gamma = torch.ones(d, device="cuda")
        self.decs, self.keys, self.caches, self.bytes_rank = [], [], [], 0
        # the token's embedding row: a small f32 matrix whose row 0 is fetched by the DecodeRow entry
        emb = torch.randn(8 * d, device="cuda", generator=gen)
        key += 1
        self.emb_key = key
        _lib.check(L.wv_pack_upload_dev(key, 0, 1, 0, emb.data_ptr(), 8, d, None))
        for layer in range(self.layers):
            keys = {}
            for pname in PROJ:
                key += 1
                r, c = shapes[pname]
                self.bytes_rank += _pack_rows(torch, L, _lib, key, 8, r, c, plan[pname][0], plan[pname][1], gen)
                keys[pname] = key
            ck = torch.randn(msl, kd, device="cuda", generator=gen)
            cv = torch.randn(msl, kd, device="cuda", generator=gen)
            self.caches.append((ck, cv))
            ptrs = {n: t.data_ptr() for n, t in self.local.items()}
            ptrs.update(attn_norm=self.gamma.data_ptr(), ffn_norm=self.gamma.data_ptr(), cache_k=ck.data_ptr(), cache_v=cv.data_ptr())
            self.decs.append(ShardedBlockDecoder(cfg, keys, ptrs, rank, world, self.vec, self.flags))
            self.keys.append(keys)
        self.heads = {}
        self.h0, self.h1 = vocab * rank // world, vocab * (rank + 1) // world
        for hname, hfmt in head_formats:
            key += 1
            self.heads[hname] = (key, hfmt, _pack_rows(torch, L, _lib, key, hfmt, vocab, d, self.h0, self.h1, gen))
        self.last_key = key
        self.pick = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.flags_all = (C.c_void_p * world)(*self.flags.ptrs) if world > 1 else None
        self.logits_all = self.vec.pointers(self.logits_off)
        torch.cuda.synchronize()
        self.setup_s = time.perf_counter() - t0

    def sync(self, st):
        if self.sworld > 1:
            self._lib.check(self.L.wv_gather_sync(self.flags_all, self.sworld, self.srank, st))

    def token(self, st, head=None, flags=True, blocks=None):
        L, chk, cfg, d = self.L, self._lib.check, self.cfg, self.cfg.DModel
        ha = self.vec.own + 4 * self.lay["ha"]
        chk(L.wv_decode_row_dev(self.emb_key, 0, ha, st))
        for dec in self.decs[:blocks]:
            dec.step(CTX, st, flags)
        if head is None:
            return
        from welvet_b200.decode import MatVecFusedCUDA        # final RMSNorm in the LM head's prologue
        MatVecFusedCUDA((C.c_uint64 * 1)(self.heads[head][0]), ha, self.logits_all, d, (C.c_int * 1)(self.h1 - self.h0),
                        dnorm_gamma=self.gamma.data_ptr(), norm_eps=cfg.Eps, world=self.sworld, rank=self.srank,
                        row_offset=(C.c_int * 1)(self.h0), stream=st)
        if flags:
            self.sync(st)
        chk(L.wv_argmax_dev(self.vec.own + 4 * self.logits_off, self.m["vocab"], self.pick.data_ptr(), st))

    def launches_per_token(self):
        return 1 + self.layers * self.decs[0].launches_per_step() + (3 if self.sworld > 1 else 2)

    def hidden(self):
        return self.vec.read(self.lay["ha"], self.cfg.DModel)

    def close(self):
        for keys in self.keys:
            for k in keys.values():
                self.L.wv_blob_evict(k)
        self.L.wv_blob_evict(self.emb_key)
        for k, _, _ in self.heads.values():
            self.L.wv_blob_evict(k)
        self.decs, self.caches = [], []


def _timed_graph(torch, stream, dist, fn, reps=5):
    """Run fn once (first launches set kernel attributes), capture it, time the replays on the device; max over ranks."""
    with torch.cuda.stream(stream):
        fn(stream.cuda_stream)
    stream.synchronize()
    if dist is not None:
        dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        fn(torch.cuda.current_stream().cuda_stream)
    if dist is not None:
        dist.barrier()
    ms = time_graph(torch, stream, g, reps)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    del g
    return ms


def _allsum(torch, dist, v):
    if dist is None:
        return v
    t = torch.tensor([float(v)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t)
    return float(t.item())


def decode_tokens(torch, L, _lib, stream, stack, dist):
    """tokens/s of the stack per LM-head format: one CUDA graph per token; sharded runs are also timed without the
    signal / wait kernels (the ranks then run unordered and the values are not meaningful) to show what the ordering costs."""
    out = {"model": "%d blocks (d_model %d, %d/%d heads of %d, FFN %d), LM head %dx%d; position %d over a cache of %d positions" % (
               stack.layers, stack.cfg.DModel, stack.cfg.NumHeads, stack.cfg.NumKVHeads, stack.cfg.HeadDim, stack.cfg.IntermediateDim,
               stack.m["vocab"], stack.cfg.DModel, CTX, CTX),
           "format": "Q4_K", "weights": "N(0,0.02^2) seed %d, every block its own matrices and caches" % stack.m["seed"],
           "setup_s": round(stack.setup_s, 1), "launches_per_token": stack.launches_per_token(), "heads": {}}
    for hname, (hkey, hfmt, hbytes) in stack.heads.items():
        row = {}
        ms = _timed_graph(torch, stream, dist, lambda st: stack.token(st, hname, True))
        row["ms_per_token"] = round(ms, 4)
        row["tokens_per_s"] = round(1e3 / ms, 2)
        tok_bytes = _allsum(torch, dist, stack.bytes_rank + hbytes)
        row["packed_bytes_per_token"] = int(tok_bytes)
        row["gbs"] = round(tok_bytes / ms / 1e6, 1)
        row["pick"] = int(stack.pick.item())
        if stack.sworld > 1:
            ms2 = _timed_graph(torch, stream, dist, lambda st: stack.token(st, hname, False))
            row["ms_per_token_without_flag_kernels"] = round(ms2, 4)
            row["ordering_ms"] = round(ms - ms2, 4)
        out["heads"][hname] = row
    out["device_status"] = int(L.wv_device_status())
    return out


def lm_head_sweep(torch, L, _lib, stream, stack, dist):
    """The row-sharded LM head alone (128256 x d_model), per format: a graph of back-to-back launches rotating over
    enough device copies of this rank's rows that no launch reads L2-resident weights; sharded, every launch is
    followed by the arrival flags, and a second timing leaves them out."""
    m, d, vocab = stack.m, stack.cfg.DModel, stack.m["vocab"]
    x = torch.randn(d, device="cuda")
    res = {}
    key = stack.last_key + 0x1000
    for hname, (hkey, hfmt, hbytes) in stack.heads.items():
        K = max(1, int(np.ceil(300e6 / hbytes)))
        keys = [hkey]
        gen = torch.Generator(device="cuda")
        for k in range(1, K):
            gen.manual_seed(1000 + k)
            key += 1
            _pack_rows(torch, L, _lib, key, hfmt, vocab, d, stack.h0, stack.h1, gen)
            keys.append(key)
        n_l = max(8, 4 * K)

        def run(st, flags):
            for i in range(n_l):
                _lib.check(L.wv_matvec_dev_gather(keys[i % K], x.data_ptr(), stack.logits_all, stack.sworld, stack.srank, stack.h0, d,
                                                  stack.h1 - stack.h0, st))
                if flags:
                    stack.sync(st)
        us = _timed_graph(torch, stream, dist, lambda st: run(st, True)) / n_l * 1e3
        full = _allsum(torch, dist, hbytes)
        row = {"rows": vocab, "cols": d, "packed_bytes": int(full), "us": round(us, 2), "gbs": round(full / us / 1e3, 1),
               "frac_8TBs_per_gpu": round(full / us / 1e3 / NOMINAL_HBM_GBS / stack.world, 3), "copies_rotated": K}
        if stack.sworld > 1:
            us2 = _timed_graph(torch, stream, dist, lambda st: run(st, False)) / n_l * 1e3
            row["us_kernel_only"] = round(us2, 2)
            row["us_ordering"] = round(us - us2, 2)
        for k in keys[1:]:
            L.wv_blob_evict(k)
        res[hname] = row
    return res


def block0_parity(torch, L, _lib, O, stack):
    """One block of the stack against the reference's host arithmetic: float64 RMSNorm, RoPE, attention and SiLU
    product from the oracle around f32 GEMVs over the dequantised weights the device holds (whose bit-exactness
    against the oracle's Unpack the per-format table reports). Returns max |h - h_ref| / max |h_ref|."""
    from welvet_b200.decode import projection_shapes
    cfg, d = stack.cfg, stack.cfg.DModel
    shapes = projection_shapes(cfg)
    W = {}
    for pname in PROJ:
        r, c = shapes[pname]
        w = np.empty(r * c, np.float32)
        _lib.check(L.wv_unpack(stack.keys[0][pname], w.ctypes.data))
        W[pname] = w.reshape(r, c)
    x = np.empty(d, np.float32)
    _lib.check(L.wv_decode_row(stack.emb_key, 0, x.ctypes.data, d))
    ck, cv = (t.cpu().numpy().astype(np.float64) for t in stack.caches[0])
    g = np.ones(d, np.float32)
    n1 = O.rmsnorm(x, g)
    q, k, v = (W[n] @ n1 for n in ("q", "k", "v"))
    qr = O.rope(q, CTX, cfg.NumHeads, cfg.HeadDim)
    ck[CTX % cfg.MaxSeqLen] = O.rope(k, CTX, cfg.NumKVHeads, cfg.HeadDim)
    cv[CTX % cfg.MaxSeqLen] = v
    attn = O.attn_decode(qr, ck, cv, cfg.NumHeads, cfg.NumKVHeads, cfg.HeadDim, CTX + 1, cfg.MaxSeqLen).astype(np.float32)
    h1 = x + W["o"] @ attn
    n2 = O.rmsnorm(h1, g)
    ref = h1 + W["down"] @ O.silu_mul(W["gate"] @ n2, W["up"] @ n2)
    stack.token(None, None, True, blocks=1)
    torch.cuda.synchronize()
    got = stack.hidden()
    return float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))


def sharded_chain_check(torch, L, _lib, stack, exchange_none, dist):
    """The sharded stack against its unsharded twin on this rank: the hidden state after two blocks must agree bit
    for bit (each output row is computed by the same code whatever rank holds it), and every rank must hold the same
    hidden state, logits and pick after a whole token."""
    twin = DecodeStack(torch, L, _lib, "70B" if stack.m is MODELS["70B"] else "8B", [], stack.rank, stack.world, None, layers=2, full_rows=True)
    twin.token(None, None, True)
    stack.token(None, None, True, blocks=2)
    torch.cuda.synchronize()
    same = bool(np.array_equal(twin.hidden().view(np.uint32), stack.hidden().view(np.uint32)))
    twin.close()
    twin.vec.close()
    dist.barrier()
    hname = next(iter(stack.heads))
    stack.token(None, hname, True)
    torch.cuda.synchronize()
    dist.barrier()
    logits = torch.from_numpy(stack.vec.read(stack.logits_off, stack.m["vocab"])).cuda()
    mine = torch.cat([torch.from_numpy(stack.hidden()).cuda(), logits, stack.pick.float()])
    ref = mine.clone()
    dist.broadcast(ref, 0)
    same = same and bool(torch.equal(mine.view(torch.int32), ref.view(torch.int32)))
    t = torch.tensor([1.0 if same else 0.0], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item() == 1.0)


def small_batch_gemm(torch, L, _lib, stream, O):
    """M activation rows x 4096 against W 4096 x 4096 (N(0, 0.02^2) seed 3) packed as Q8_0 and as the 4-bit k-quant,
    M in {1, 4, 16, 64, 256}: one wv_matvec_dev call per M, rotating over enough device copies of W that no launch
    reads L2-resident weights. Small batches of this L2-sized matrix run row by row on the batch-1 kernel, larger
    ones on the tcgen05 kernel that dequantises W once per call; parity of the first and last row against the oracle."""
    rows = cols = 4096
    rng = np.random.default_rng(3)
    w_host = rng.normal(0, 0.02, rows * cols).astype(np.float32)
    x_host = rng.normal(0, 1, (256, cols)).astype(np.float32)
    w = torch.from_numpy(w_host).cuda()
    x = torch.from_numpy(x_host).cuda()
    out = {"shape": "M x 4096 times W 4096 x 4096, weights N(0,0.02^2) seed 3", "cases": []}
    key0 = 0x300000
    for name, fmt in (("Q8_0", 1), ("Q4_K", 8)):
        _lib.check(L.wv_pack_upload_dev(key0, fmt, 1, 0, w.data_ptr(), rows, cols, None))
        wb = C.c_uint64()
        _lib.check(L.wv_blob_info(key0, None, None, C.byref(wb), None, None))
        nbytes = int(wb.value)
        K = max(2, int(np.ceil(300e6 / nbytes)))
        keys = [key0]
        for k in range(1, K):
            _lib.check(L.wv_pack_upload_dev(key0 + k, fmt, 1, 0, w.data_ptr(), rows, cols, None))
            keys.append(key0 + k)
        ob = O.pack(name, w_host, rows, cols) if O is not None else None
        for M in (1, 4, 16, 64, 256):
            y = torch.zeros(M, rows, device="cuda")
            n_l = 2 * K

            def run(st):
                for i in range(n_l):
                    _lib.check(L.wv_matvec_dev(keys[i % K], x.data_ptr(), y.data_ptr(), M, cols, rows, st))
            us = _timed_graph(torch, stream, None, run) / n_l * 1e3
            row = {"format": name, "M": M, "us": round(us, 2), "gbs_packed_weights": round(nbytes / us / 1e3, 1),
                   "tflops": round(2.0 * M * rows * cols / us / 1e6, 2),
                   "kernel": "tcgen05 (TF32 operands, W dequantised once)" if M >= 6 else "batch-1 integer-dot kernel, one launch per row"}
            if ob is not None:
                got = y.cpu().numpy()
                worst = 0.0
                for m in sorted({0, M - 1}):
                    ref = O.matvec_simd(ob, x_host[m], 0).astype(np.float64)
                    den = O.sum_abs_wx(ob, x_host[m])
                    worst = max(worst, float(np.max(np.abs(got[m].astype(np.float64) - ref) / np.maximum(den, 1e-30))))
                row["max_rel"] = float(f"{worst:.3e}")
            out["cases"].append(row)
        for k in keys:
            L.wv_blob_evict(k)
        key0 += 0x100
    out["roofline_note"] = ("HBM roofline for M <= 16 (W streamed once: 18.9 MB Q8_0, 11.0 MB Q4_K); for M >= 64 the TF32 tensor pipe "
                            "(dense TF32 is half the bf16 rate) next to the same weight stream")
    return out


def size_sweep(torch, L, _lib, stream):
    """Launch time against matrix size for three formats (same timing method as the per-format table): the least-squares
    line t = fixed + bytes / rate separates the per-launch overhead from the streaming rate."""
    shapes = [(2368, 14336), (4096, 14336), (8192, 8192), (14336, 8192), (28672, 8192), (65536, 8192)]
    out = {}
    key = 0x600000
    for name, fmt in (("Q4_0", 2), ("Q4_K", 8), ("Q8_0", 1)):
        pts = []
        for rows, cols in shapes:
            w = torch.randn(rows * cols, device="cuda") * 0.02
            x = torch.randn(cols, device="cuda")
            y = torch.zeros(rows, device="cuda")
            keys, nbytes = [], 0
            for k in range(32):
                key += 1
                _lib.check(L.wv_pack_upload_dev(key, fmt, 1, 0, w.data_ptr(), rows, cols, None))
                wb = C.c_uint64()
                _lib.check(L.wv_blob_info(key, None, None, C.byref(wb), None, None))
                nbytes = int(wb.value)
                keys.append(key)
                if len(keys) * nbytes >= 300e6 and len(keys) >= 2:
                    break
            K, n_l = len(keys), 4 * len(keys)

            def run(st):
                for i in range(n_l):
                    _lib.check(L.wv_matvec_dev(keys[i % K], x.data_ptr(), y.data_ptr(), 1, cols, rows, st))
            us = _timed_graph(torch, stream, None, run) / n_l * 1e3
            pts.append({"rows": rows, "cols": cols, "packed_bytes": nbytes, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1)})
            for k in keys:
                L.wv_blob_evict(k)
            del w
        b = np.array([p["packed_bytes"] for p in pts], np.float64)
        t = np.array([p["us"] for p in pts], np.float64)
        slope, fixed = np.polyfit(b, t, 1)
        out[name] = {"points": pts, "fixed_us": round(float(fixed), 2), "streaming_gbs": round(1e-3 / float(slope), 1)}
    return out


def run_decode_configs(torch, L, _lib, stream, rank, world, exchange, dist):
    """The decode configurations beside the headline sweep: the 8B stack on one GPU (tokens/s, one block checked against
    the reference's host arithmetic) and the 70B stack with its LM head as Q8_0 and Q4_K, row-sharded over the ranks."""
    res = {}
    if world == 1:
        st8 = DecodeStack(torch, L, _lib, "8B", [("Q4_K", 8)], 0, 1, None)
        c4 = decode_tokens(torch, L, _lib, stream, st8, None)
        import oracle as O
        c4["block0_max_rel_vs_host_arithmetic"] = float("%.3e" % block0_parity(torch, L, _lib, O, st8))
        st8.close()
        st8.vec.close()
        del st8
        torch.cuda.empty_cache()
        res["config4"] = c4
    st70 = DecodeStack(torch, L, _lib, "70B", [("Q8_0", 1), ("Q4_K", 8)], rank, world, exchange)
    c5 = {"n_gpus": world, "lm_head": lm_head_sweep(torch, L, _lib, stream, st70, dist),
          "stack": decode_tokens(torch, L, _lib, stream, st70, dist),
          "sharding": "rows of every projection and of the LM head split evenly over the ranks; each rank's kernels store their rows into "
                      "every rank's vectors over NVLink (peer mappings), ordered by arrival flags on the device; norms, RoPE, the cache "
                      "and attention run replicated" if world > 1 else "single GPU"}
    if world > 1:
        c5["sharded_equals_unsharded"] = sharded_chain_check(torch, L, _lib, st70, None, dist)
        torch.cuda.synchronize()
        dist.barrier()
        st70.vec.close_peers()
        st70.flags.close_peers()
        torch.cuda.synchronize()
        dist.barrier()
    st70.close()
    st70.vec.free_own()
    if st70.flags is not None:
        st70.flags.free_own()
    res["config5"] = c5
    return res


def main():
    # stdout carries the one JSON line and nothing else: libraries that print there (NCCL's version
    # banner, for one) are sent to stderr, the line itself goes to the saved descriptor
    global _STDOUT_FD
    sys.stdout.flush()
    _STDOUT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="welvet_b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the per-format parity fields")
    ap.add_argument("--e2e-callers", type=int, default=4, help="caller threads of the end-to-end measurement (the library has eight staging slots)")
    ap.add_argument("--size-sweep", action="store_true", help="only: launch time against matrix size for Q4_0 / Q4_K / Q8_0 (prints its own JSON line)")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-stack decode runs (8B block stack, 70B row-sharded stack and LM head)")
    ap.add_argument("--formats", default="", help="comma list: restrict the sweep (for profiler captures)")
    ap.add_argument("--quick", action="store_true", help="skip the per-format table, the e2e and the CPU legs (profiler captures)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)
    sweep = [f for f in SWEEP if not args.formats or f[0] in args.formats.split(",")]
    if args.formats:       # a restricted run (profiler captures) may also name the formats measured outside the step
        sweep += [f for f in EXTRA if f[0] in args.formats.split(",")]
    extra = [] if (args.formats or args.quick) else EXTRA

    import torch
    import welvet_b200 as wv
    from welvet_b200 import _lib
    torch.cuda.set_device(local)
    wv.init(local)
    L = _lib.lib()
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    stream = torch.cuda.Stream()
    if args.size_sweep:
        if rank == 0:
            emit({"size_sweep": size_sweep(torch, L, _lib, stream), "unit": "us per launch; GB/s of packed weight bytes", "n_gpus": 1})
        return

    # ---- build the sweep on the device (device packer == reference packer, byte for byte)
    jobs = []
    extra_jobs = []
    xs, xh, wh = {}, {}, {}
    nkey = 0x10000
    for rows, cols in SHAPES:
        wh[cols] = gen_weights(rows, cols)
        w = torch.from_numpy(wh[cols]).cuda()
        xh[cols] = gen_x(cols)
        xs[cols] = torch.from_numpy(xh[cols]).cuda()
        lo, hi = C.c_int(), C.c_int()
        _lib.check(L.wv_shard_range(rows, rank, world, C.byref(lo), C.byref(hi)))
        r0, r1 = lo.value, hi.value
        for group, lst in ((jobs, sweep), (extra_jobs, extra if world == 1 else [])):
            for spec in lst:
                name, fmt, bw, dt = spec
                nkey += 1
                _lib.check(L.wv_pack_upload_dev(nkey, fmt, dt, bw, w.data_ptr() + r0 * cols * 4, r1 - r0, cols, None))
                wb = C.c_uint64()
                _lib.check(L.wv_blob_info(nkey, None, None, C.byref(wb), None, None))
                y = torch.zeros(rows, device="cuda")
                group.append(dict(name=name, spec=spec, key=nkey, rows=rows, cols=cols, r0=r0, r1=r1, bytes=int(wb.value), y=y))
        del w
    torch.cuda.synchronize()

    # N > 1: every rank owns a row range of every matrix and its kernels store their rows into
    # all ranks' output vectors (peer mappings of one exportable buffer per rank): the gather is
    # the GEMV's epilogue, there is no collective call inside the step and the step stays a graph.
    gbufs = None
    if world > 1:
        from welvet_b200.dense import GatherBuffers

        def exchange(h):
            out = [None] * world
            dist.all_gather_object(out, h)
            return out
        off = 0
        for j in jobs:
            j["off"] = off
            off += j["rows"]
        gbufs = GatherBuffers(4 * off, rank, world, exchange)
        gflags = GatherBuffers(4 * (world + 2), rank, world, exchange)
        f_all = (C.c_void_p * world)(*gflags.ptrs)
        for j in jobs:
            j["y_all"] = gbufs.pointers(j["off"])

    def launch(j, st):
        if world > 1:
            _lib.check(L.wv_matvec_dev_gather(j["key"], xs[j["cols"]].data_ptr(), j["y_all"], world, rank, j["r0"], j["cols"], j["r1"] - j["r0"], st))
        else:
            _lib.check(L.wv_matvec_dev(j["key"], xs[j["cols"]].data_ptr(), j["y"].data_ptr(), 1, j["cols"], j["rows"], st))

    def step_end(st):
        # a step is complete on a rank when every rank's rows have arrived: arrival flags, on the device
        if world > 1:
            _lib.check(L.wv_gather_signal(f_all, world, rank, st))
            _lib.check(L.wv_gather_wait(gflags.own, world, st))

    with torch.cuda.stream(stream):
        for j in jobs:                     # first call per kernel sets its attributes (not capturable)
            launch(j, stream.cuda_stream)
        step_end(stream.cuda_stream)
    stream.synchronize()
    # One CUDA graph per step: the 38 GEMV launches (and, sharded, the two flag kernels), at every N.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        cur = torch.cuda.current_stream().cuda_stream
        for j in jobs:
            launch(j, cur)
        step_end(cur)

    # The step graph is replayed R times per step so that the timed region lasts at least MIN_TIMED_S
    # (20 steps of 0.3 ms would be 6 ms: too short for a clock sample); the time is divided by K * R.
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            graph.replay()
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream); graph.replay(); b.record(stream)
        stream.synchronize()
        probe_ms = a.elapsed_time(b)
    reps = max(1, int(np.ceil(MIN_TIMED_S * 1e3 / max(probe_ms * args.steps, 1e-3))))
    if world > 1:
        t = torch.tensor([float(reps)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        reps = int(t.item())
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(args.steps * reps):
            graph.replay()
        e1.record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop() if sampler else None
    ms_step = ms / (args.steps * reps)
    full_bytes = sum(j["bytes"] for j in jobs)
    if world > 1:
        t = torch.tensor([float(full_bytes)], device="cuda")
        dist.all_reduce(t)
        full_bytes = float(t.item())
    value = full_bytes / (ms_step * 1e-3) / 1e9
    launches_per_step = len(jobs) + (2 if world > 1 else 0)   # one launch per GEMV (+ the two flag kernels of a sharded step)

    gather_ok = None
    if world > 1:
        # the gathered vectors must equal the unsharded product's, bit for bit: every job, on every rank
        torch.cuda.synchronize()
        dist.barrier()
        ok = True
        for j in jobs:
            w = torch.from_numpy(wh[j["cols"]]).cuda()
            spec = j["spec"]
            _lib.check(L.wv_pack_upload_dev(0x7FFF01, spec[1], spec[3], spec[2], w.data_ptr(), j["rows"], j["cols"], None))
            ref = torch.zeros(j["rows"], device="cuda")
            _lib.check(L.wv_matvec_dev(0x7FFF01, xs[j["cols"]].data_ptr(), ref.data_ptr(), 1, j["cols"], j["rows"], None))
            torch.cuda.synchronize()
            got = gbufs.read(j["off"], j["rows"])
            ok = ok and bool(np.array_equal(got.view(np.uint32), ref.cpu().numpy().view(np.uint32)))
            L.wv_blob_evict(0x7FFF01)
            del w
        t = torch.tensor([1.0 if ok else 0.0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        gather_ok = bool(t.item() == 1.0)
        # unmap the peers' buffers everywhere before any rank frees its own, then leave together
        graph = None
        if L.wv_device_status() != 0:
            gather_ok = False
        gbufs.close_peers()
        gflags.close_peers()
        torch.cuda.synchronize()
        dist.barrier()
        gbufs.free_own()
        gflags.free_own()
        for j in jobs:
            L.wv_blob_evict(j["key"])
        decode = None
        if not args.quick and not args.formats and not args.no_decode:
            decode = run_decode_configs(torch, L, _lib, stream, rank, world, exchange, dist)
        dist.destroy_process_group()
    if rank != 0:
        return

    # ---- per-format kernel times, measured live: a CUDA graph of back-to-back launches of the one
    # kernel, rotating over K device copies of the blob (K * bytes >= 300 MB, more than twice L2) so
    # that no launch reads L2-resident weights; CUDA events on the launching stream. Beside each time:
    # the parity of that very blob and output against the oracle (dequant bit-exact, max relative error).
    peak, peak_src = measured_hbm_peak()
    per = []
    if world == 1 and not args.quick:
        O = None
        scratch = None
        if not args.no_parity:
            import oracle as O
            scratch = torch.empty(max(r * c for r, c in SHAPES), device="cuda")
        last_cols, w = None, None
        for j in jobs + extra_jobs:
            K = max(2, min(32, int(np.ceil(300e6 / j["bytes"]))))
            keys = [j["key"]]
            rows, cols = j["rows"], j["cols"]
            if cols != last_cols:
                w = torch.from_numpy(wh[cols]).cuda()
            last_cols = cols
            spec = j["spec"]
            for k in range(1, K):
                nkey += 1
                _lib.check(L.wv_pack_upload_dev(nkey, spec[1], spec[3], spec[2], w.data_ptr(), rows, cols, None))
                keys.append(nkey)
            with torch.cuda.stream(stream):
                for k in keys:   # first launch of a kernel sets its attributes
                    _lib.check(L.wv_matvec_dev(k, xs[cols].data_ptr(), j["y"].data_ptr(), 1, cols, rows, stream.cuda_stream))
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            n_l = 4 * K
            with torch.cuda.graph(g, stream=stream):
                cur = torch.cuda.current_stream().cuda_stream
                for i in range(n_l):
                    _lib.check(L.wv_matvec_dev(keys[i % K], xs[cols].data_ptr(), j["y"].data_ptr(), 1, cols, rows, cur))
            us = time_graph(torch, stream, g) / n_l * 1e3
            del g
            for k in keys[1:]:
                L.wv_blob_evict(k)
            gbs = j["bytes"] / us / 1e3
            row = {"format": j["name"], "rows": rows, "cols": cols, "packed_bytes": j["bytes"], "us": round(us, 2),
                   "gbs": round(gbs, 1), "frac_measured_peak": round(gbs / peak, 3), "frac_8TBs": round(gbs / NOMINAL_HBM_GBS, 3),
                   "copies_rotated": K, "in_step": j in jobs}
            if O is not None:
                exact, rel = parity_sample(torch, L, _lib, O, spec, wh[cols], xh[cols], rows, cols, j["key"], j["y"], scratch)
                row["dequant_bitexact"] = exact
                row["max_rel"] = float(f"{rel:.3e}")
            per.append(row)
        del w, scratch
    # The step is 38 launches of one kernel family (a template instance per format); none of them
    # dominates, so the roofline is taken over the family: bytes per launch and launch duration
    # are the averages over the step's launches, each timed in its own same-kernel graph above.
    in_step = [p for p in per if p["in_step"]]
    dom = None
    if in_step:
        fam_bytes = sum(p["packed_bytes"] for p in in_step) / len(in_step)
        fam_us = sum(p["us"] for p in in_step) / len(in_step)
        ratio = sum(NCU_DRAM_BYTES.values()) / sum(NCU_ALGO_BYTES.values())
        dom = {"gbs": fam_bytes / fam_us / 1e3, "bytes": fam_bytes, "us": fam_us, "traffic": int(fam_bytes * ratio),
               "slow": max(in_step, key=lambda p: p["us"]), "fast": max(in_step, key=lambda p: p["gbs"])}

    # ---- end to end through the host-pointer plugin call
    yh = {j["key"]: np.zeros(j["r1"] - j["r0"], np.float32) for j in jobs}

    def e2e_call(j):
        _lib.check(L.wv_matvec(j["key"], xh[j["cols"]].ctypes.data, yh[j["key"]].ctypes.data, 1, j["cols"], j["r1"] - j["r0"]))

    def e2e_run(callers, passes):
        """Seconds per pass over the sweep with `callers` threads, each making the calls of its own share of the
        matrices (every thread loops in its own right: a task queue between Python threads costs more per call
        than the call)."""
        import threading
        shares = [jobs[i::callers] for i in range(callers)]
        gate = threading.Barrier(callers + 1)
        errs = []

        def work(mine):
            try:
                for _ in range(3):                 # warm: the thread's staging slot and its launch graphs
                    for j in mine:
                        e2e_call(j)
                gate.wait()
                for _ in range(passes):
                    for j in mine:
                        e2e_call(j)
            except Exception as ex:                # noqa: BLE001 - reported by the caller below
                errs.append(ex)
                gate.abort()
        th = [threading.Thread(target=work, args=(m,)) for m in shares]
        for t in th:
            t.start()
        try:
            gate.wait()
        except threading.BrokenBarrierError:
            pass
        t0 = time.perf_counter()
        for t in th:
            t.join()
        dt = time.perf_counter() - t0
        if errs:
            raise errs[0]
        return dt / passes
    e2e_val, e2e_single = None, None
    E2E_CALLERS = args.e2e_callers
    if world == 1 and not args.quick:
        # Every call is the synchronous host-pointer plugin call (x copied in, y copied out inside it). The headline figure
        # has several caller threads in flight (four by default), as the reference's Dense is called from several goroutines
        # (layers/dense/cpu.go forwardTiledMC) and as the library's eight staging slots allow; one caller is reported beside it.
        n_e2e = max(args.steps, 20)
        for callers in sorted({1, max(1, E2E_CALLERS)}):
            e2e_s = e2e_run(callers, n_e2e)
            if callers > 1:
                e2e_val = full_bytes / e2e_s / 1e9
            else:
                e2e_single = full_bytes / e2e_s / 1e9
                if E2E_CALLERS <= 1:
                    e2e_val = e2e_single

    cfg = common_config(sweep)
    out = {
        "metric": METRIC,
        "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8x4 dot (block-fixed-point activations) + f32 scale",
        "data": "synthetic",
        "config": cfg,
        "run": {"replays_per_step": reps, "timed_region_s": round(ms * 1e-3, 4), "launch": "cuda graph of the step",
                "pct_of_8TBs": round(100 * value / NOMINAL_HBM_GBS, 1),
                "sharding": ("rows split evenly across ranks; each rank's GEMV kernels store their rows into every rank's y "
                             "(peer mappings, no collective call); every step ends with on-device arrival flags; "
                             "gathered y verified bit-identical to the unsharded product on all %d jobs: %s" % (len(jobs), gather_ok))
                if world > 1 else "single GPU"},
        "gpu_launches": launches_per_step * args.steps * reps,
        "clocks": clocks,
    }
    if dom:
        def brief(p):
            return {"format": p["format"], "shape": f'{p["rows"]}x{p["cols"]}', "us": p["us"], "gbs": p["gbs"],
                    "frac": round(p["gbs"] / peak, 3)}
        out["roofline"] = {"bound": "hbm", "kernel": f"batch-1 GEMV kernel family, {len(in_step)} launches per step",
                           "achieved": round(dom["gbs"], 1), "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                           "frac": round(dom["gbs"] / peak, 3), "traffic": dom["traffic"],
                           "bytes_per_launch": int(dom["bytes"]), "us_per_launch": round(dom["us"], 2),
                           "traffic_note": "average algorithmic bytes per launch x the ncu DRAM/algorithmic ratio of captured Q4_0, Q8_0, Q4_K, Q5_K, Q2_K, IQ4_NL launches",
                           "slowest": brief(dom["slow"]), "fastest": brief(dom["fast"])}
        out["per_format"] = per
        if any("dequant_bitexact" in p for p in per):
            out["parity"] = {"dequant_bitexact_all": all(p.get("dequant_bitexact", True) for p in per),
                             "max_rel_worst": max(p.get("max_rel", 0.0) for p in per), "tolerance": 1e-3,
                             "rows_checked": "three 64-row bands (first, middle, last) of every matrix"}
    if e2e_val is not None:
        out["e2e"] = {"value": e2e_val, "unit": "GB/s", "callers": E2E_CALLERS, "value_one_caller": e2e_single,
                      "h2d_bytes_per_step": int(sum(4 * j["cols"] for j in jobs)),
                      "d2h_bytes_per_step": int(sum(4 * (j["r1"] - j["r0"]) for j in jobs))}
    if world == 1 and not args.no_cpu_baseline and not args.quick:
        sample = [f for f in SWEEP if f[0] in ("Q4_0", "Q8_0", "Q4_K", "Q6_K", "IQ3_S", "TernaryPacked", "BinaryPacked_g128")]
        gbs, cores, sec, total = cpu_leg(3, 1, sample, SHAPES[:1])
        out["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                               "sample": f"{len(sample)} formats ({','.join(f[0] for f in sample)}) at 4096x14336, 3 timed passes, SIMD-path caches prebuilt"}
    if world == 1 and not args.quick and not args.formats and not args.no_decode:
        for j in jobs + extra_jobs:
            L.wv_blob_evict(j["key"])
        decode = run_decode_configs(torch, L, _lib, stream, 0, 1, None, None)
        O3 = None
        if not args.no_parity:
            import oracle as O3
        decode["config3"] = small_batch_gemm(torch, L, _lib, stream, O3)
    if not args.quick and not args.formats and not args.no_decode:
        out.update(decode)
    emit(out)


if __name__ == "__main__":
    main()
