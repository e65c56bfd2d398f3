"""Single-token decode of one decoder block with every step on the device: the reference's
block walk (model/transformer/forward.go:57-76: RMSNorm -> attention -> residual -> RMSNorm ->
SwiGLU -> residual) with its host-side float64 steps (layers/rmsnorm/cpu.go, layers/mha/cpu.go,
layers/mha/rope.go, layers/mha/attn.go, layers/swiglu/cpu.go) replaced by the device entries of
include/welvet_cuda.h, so that activations stay in HBM between the projection GEMVs.

All pointers are device addresses (ints); the caller owns the buffers (for example torch tensors)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

from . import quant
from ._lib import check, lib


def RMSNormCUDA(dx: int, dgamma: int, dy: int, rows: int, dim: int, eps: float, stream: int = 0) -> None:
    """rmsnorm.Forward post output (layers/rmsnorm/cpu.go:32-90) for float32 rows."""
    check(lib().wv_rmsnorm_dev(dx, dgamma, dy, rows, dim, eps, stream))


def RoPECacheCUDA(dq: int, dk: int, dv: int, dcache_k: int, dcache_v: int, pos: int, max_seq_len: int, num_heads: int,
                  num_kv_heads: int, head_dim: int, theta: float, stream: int = 0) -> None:
    """applyRoPE on Q (in place) and K, K and V into cache row pos % max_seq_len (mha/rope.go:6-21, mha/cpu.go:184-207)."""
    check(lib().wv_rope_cache_dev(dq, dk, dv, dcache_k, dcache_v, pos, max_seq_len, num_heads, num_kv_heads, head_dim, theta, stream))


def AttnDecodeCUDA(dq: int, dcache_k: int, dcache_v: int, dout: int, num_heads: int, num_kv_heads: int, head_dim: int, kv_len: int,
                   max_seq_len: int, scale: float, stream: int = 0) -> None:
    """attnForward for one query token under the causal mask (mha/attn.go:15-120)."""
    check(lib().wv_attn_decode_dev(dq, dcache_k, dcache_v, dout, num_heads, num_kv_heads, head_dim, kv_len, max_seq_len, scale, stream))


def SiluMulCUDA(dgate: int, dup: int, dout: int, n: int, stream: int = 0) -> None:
    """simd.SiluMulF32 (simd/silu.go:7-27)."""
    check(lib().wv_silu_mul_dev(dgate, dup, dout, n, stream))


def ResidualAddCUDA(ddst: int, dadd: int, n: int, stream: int = 0) -> None:
    """residualAddInPlace (model/transformer/scratch.go:33-41)."""
    check(lib().wv_residual_add_dev(ddst, dadd, n, stream))


def MatVecSwiGLUCUDA(key_gate: int, key_up: int, dx: int, dh: int, in_: int, out: int, stream: int = 0) -> None:
    """h = silu(W_gate x) * (W_up x) in one launch (swiglu/cpu.go:29-52, fusedgpu/shaders.go:159-222)."""
    check(lib().wv_matvec_dev_swiglu(key_gate, key_up, dx, dh, in_, out, stream))


def MatVecAddCUDA(key: int, dx: int, dresidual: int, dy: int, in_: int, out: int, stream: int = 0) -> None:
    """y = W x + residual in one launch (forward.go:65,75; fusedgpu/hybrid_shaders.go:82)."""
    check(lib().wv_matvec_dev_add(key, dx, dresidual, dy, in_, out, stream))


def MatVecFusedCUDA(keys, dx: int, y_all, in_: int, out_local, mode: int = 0, dresidual: Optional[int] = None,
                    dnorm_gamma: Optional[int] = None, norm_eps: float = 0.0, world: int = 1, rank: int = 0, row_offset=None,
                    stream: int = 0) -> None:
    """wv_matvec_dev_fused: up to four projections on a shared x in one launch, with the RMSNorm of x in the prologue
    and the SiLU product / residual add / stores to every rank's vectors in the epilogue, as requested.
    keys, y_all, out_local, row_offset are ctypes arrays (uint64, void*, int, int)."""
    from ._lib import WvFusedCall
    call = WvFusedCall(keys, len(keys), dx, y_all, world, rank, row_offset, in_, out_local, mode, dresidual, dnorm_gamma, norm_eps)
    check(lib().wv_matvec_dev_fused(C.byref(call), stream))


@dataclass
class BlockConfig:
    """Shape of one decoder block (mha.Config / swiglu.Config fields the decode path uses)."""
    DModel: int
    NumHeads: int
    NumKVHeads: int
    HeadDim: int
    IntermediateDim: int
    MaxSeqLen: int
    Eps: float = 1e-5
    RoPETheta: float = 10000.0


class BlockDecoder:
    """One block's single-token decode as seven launches: Q|K|V group with the attention RMSNorm in its prologue, RoPE +
    cache write, attention (splits, then their merge), O + residual, gate|up with the FFN RMSNorm in its prologue and the
    SiLU product in its epilogue, down + residual. `keys` maps
    q, k, v, o, gate, up, down to resident blob keys; `bufs` maps the working vectors (q, k, v,
    attn, ffn) and the weights attn_norm / ffn_norm and caches cache_k / cache_v to device pointers."""

    def __init__(self, cfg: BlockConfig, keys: dict, bufs: dict):
        self.cfg, self.keys, self.bufs = cfg, keys, bufs
        c = cfg
        self._qkv_keys = (C.c_uint64 * 3)(keys["q"], keys["k"], keys["v"])
        self._qkv_outs = (C.c_int * 3)(c.NumHeads * c.HeadDim, c.NumKVHeads * c.HeadDim, c.NumKVHeads * c.HeadDim)
        self._qkv_ptrs = (C.c_void_p * 3)(bufs["q"], bufs["k"], bufs["v"])
        self._gu_keys = (C.c_uint64 * 2)(keys["gate"], keys["up"])
        self._gu_outs = (C.c_int * 2)(c.IntermediateDim, c.IntermediateDim)
        self._gu_ptrs = (C.c_void_p * 2)(None, bufs["ffn"])

    def step(self, dh: int, pos: int, stream: int = 0) -> None:
        """h (device pointer to DModel floats) is updated in place; pos is the token's position."""
        c, k, b, L = self.cfg, self.keys, self.bufs, lib()
        qd = c.NumHeads * c.HeadDim
        MatVecFusedCUDA(self._qkv_keys, dh, self._qkv_ptrs, c.DModel, self._qkv_outs, dnorm_gamma=b["attn_norm"], norm_eps=c.Eps, stream=stream)
        RoPECacheCUDA(b["q"], b["k"], b["v"], b["cache_k"], b["cache_v"], pos, c.MaxSeqLen, c.NumHeads, c.NumKVHeads, c.HeadDim, c.RoPETheta, stream)
        AttnDecodeCUDA(b["q"], b["cache_k"], b["cache_v"], b["attn"], c.NumHeads, c.NumKVHeads, c.HeadDim, min(pos + 1, c.MaxSeqLen), c.MaxSeqLen,
                       1.0 / (c.HeadDim ** 0.5), stream)
        MatVecAddCUDA(k["o"], b["attn"], dh, dh, qd, c.DModel, stream)
        MatVecFusedCUDA(self._gu_keys, dh, self._gu_ptrs, c.DModel, self._gu_outs, mode=1, dnorm_gamma=b["ffn_norm"], norm_eps=c.Eps, stream=stream)
        MatVecAddCUDA(k["down"], b["ffn"], dh, dh, c.IntermediateDim, c.DModel, stream)


PROJECTIONS = ("q", "k", "v", "o", "gate", "up", "down")


def projection_shapes(cfg: BlockConfig) -> dict:
    """rows x cols of the seven Dense projections of a block (mha.Config / swiglu.Config)."""
    qd, kd = cfg.NumHeads * cfg.HeadDim, cfg.NumKVHeads * cfg.HeadDim
    return {"q": (qd, cfg.DModel), "k": (kd, cfg.DModel), "v": (kd, cfg.DModel), "o": (cfg.DModel, qd),
            "gate": (cfg.IntermediateDim, cfg.DModel), "up": (cfg.IntermediateDim, cfg.DModel), "down": (cfg.DModel, cfg.IntermediateDim)}


def shard_plan(cfg: BlockConfig, rank: int, world: int) -> dict:
    """Row range [begin, end) of every projection that `rank` of `world` keeps (rows split evenly, as the reference
    splits rows over goroutines, layers/dense/gemv_parallel.go:24-41)."""
    return {n: (r * rank // world, r * (rank + 1) // world) for n, (r, _) in projection_shapes(cfg).items()}


def vector_layout(cfg: BlockConfig) -> dict:
    """Float offsets of the gathered vectors inside each rank's exchange buffer: q, k, v, the two hidden-state
    vectors that alternate between the attention and the FFN half of a block, and the SwiGLU product."""
    qd, kd = cfg.NumHeads * cfg.HeadDim, cfg.NumKVHeads * cfg.HeadDim
    off, out = 0, {}
    for name, n in (("q", qd), ("k", kd), ("v", kd), ("ha", cfg.DModel), ("hb", cfg.DModel), ("ffn", cfg.IntermediateDim)):
        out[name] = off
        off += (n + 63) & ~63
    out["total"] = off
    return out


class ShardedBlockDecoder:
    """BlockDecoder with every projection row-sharded over `world` ranks: each rank keeps its rows of the seven
    matrices, its GEMV kernels store their rows into every rank's vectors (peer mappings of one exchange buffer per
    rank), and arrival flags on the device order the ranks; RMSNorm, RoPE, the cache and attention are replicated.
    Four sharded launches per block (Q|K|V and gate|up with their RMSNorm in the prologue, the latter with the SiLU
    product; O and down with the residual), each followed by the signal-and-wait launch when world > 1.

    The hidden state alternates between the vectors `ha` and `hb` of the exchange buffer: a block reads `ha`, the O
    projection writes `hb`, the down projection writes `ha` again. A rank can run at most one sharded launch ahead
    of the slowest rank (it cannot pass a wait before every rank has signalled), and no launch writes a vector that
    the previous launch's consumers read, so peers never overwrite data still in use.

    keys: this rank's resident shard of q, k, v, o, gate, up, down. local: device pointers of attn and the
    weights attn_norm / ffn_norm and caches cache_k / cache_v. vec / flags: dense.GatherBuffers."""

    def __init__(self, cfg: BlockConfig, keys: dict, local: dict, rank: int, world: int, vec, flags=None):
        self.cfg, self.keys, self.local, self.rank, self.world, self.vec, self.flags = cfg, keys, local, rank, world, vec, flags
        self.off = vector_layout(cfg)
        plan = shard_plan(cfg, rank, world)
        self.plan = plan

        def arrays(names, outs):
            n = len(names)
            ptrs = []
            for o in outs:
                ptrs += [None] * world if o is None else list(vec.pointers(self.off[o]))
            return ((C.c_uint64 * n)(*[keys[m] for m in names]), (C.c_void_p * (n * world))(*ptrs),
                    (C.c_int * n)(*[plan[m][0] for m in names]), (C.c_int * n)(*[plan[m][1] - plan[m][0] for m in names]))
        self._qkv = arrays(("q", "k", "v"), ("q", "k", "v"))
        self._o = arrays(("o",), ("hb",))
        self._gu = arrays(("gate", "up"), (None, "ffn"))
        self._down = arrays(("down",), ("ha",))
        self._flags_all = (C.c_void_p * world)(*flags.ptrs) if world > 1 else None

    def _sync(self, stream: int) -> None:
        if self.world > 1:
            L = lib()
            check(L.wv_gather_sync(self._flags_all, self.world, self.rank, stream))

    def _gemv(self, a, n: int, dx: int, in_: int, mode: int, dres: Optional[int], stream: int, sync: bool, gamma: Optional[int] = None) -> None:
        MatVecFusedCUDA(a[0], dx, a[1], in_, a[3], mode, dres, gamma, self.cfg.Eps if gamma else 0.0, self.world, self.rank, a[2], stream)
        if sync:
            self._sync(stream)

    def step(self, pos: int, stream: int = 0, sync: bool = True) -> None:
        """One token: the hidden state in `ha` of every rank's exchange buffer is updated in place. sync=False leaves
        the signal / wait kernels out (timing of the launches alone; the ranks then run unordered)."""
        c, b, own, off = self.cfg, self.local, self.vec.own, self.off
        qd = c.NumHeads * c.HeadDim
        ha, hb = own + 4 * off["ha"], own + 4 * off["hb"]
        q, k, v, ffn = own + 4 * off["q"], own + 4 * off["k"], own + 4 * off["v"], own + 4 * off["ffn"]
        self._gemv(self._qkv, 3, ha, c.DModel, 0, None, stream, sync, b["attn_norm"])
        RoPECacheCUDA(q, k, v, b["cache_k"], b["cache_v"], pos, c.MaxSeqLen, c.NumHeads, c.NumKVHeads, c.HeadDim, c.RoPETheta, stream)
        AttnDecodeCUDA(q, b["cache_k"], b["cache_v"], b["attn"], c.NumHeads, c.NumKVHeads, c.HeadDim, min(pos + 1, c.MaxSeqLen), c.MaxSeqLen,
                       1.0 / (c.HeadDim ** 0.5), stream)
        self._gemv(self._o, 1, b["attn"], qd, 0, ha, stream, sync)
        self._gemv(self._gu, 2, hb, c.DModel, 1, None, stream, sync, b["ffn_norm"])
        self._gemv(self._down, 1, ffn, c.IntermediateDim, 0, hb, stream, sync)

    def launches_per_step(self) -> int:
        return 7 + (4 if self.world > 1 else 0)
