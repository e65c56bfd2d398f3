"""Host-side mirror of the reference's layers/dense call surface, with the CUDA backend
as an explicit dispatch case next to the reference's CPU / SIMD / WebGPU ones
(layers/dense/dense.go:100-112). Only the forward path exists here; the GEMV runs in
libwelvet_cuda.so and nothing falls back to the host."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

import numpy as np

from . import _lib, quant, weights
from ._lib import WelvetError, check, lib

# core.Backend (core/layer.go:125-131) plus the new value.
BackendCPUTiled, BackendSIMD, BackendWebGPU, BackendCUDA = 0, 1, 2, 3
# core.ActivationType (core/layer.go:91-98): the integer values are part of the call surface.
ActivationLinear = -1
ActivationReLU = 0
ActivationSilu = 1
ActivationGELU = 2
ActivationTanh = 3
ActivationSigmoid = 4
ActivationLeakyReLU = 5
ActivationReLU2 = 6
_ACTIVATIONS = (ActivationLinear, ActivationReLU, ActivationSilu, ActivationGELU, ActivationTanh, ActivationSigmoid,
                ActivationLeakyReLU, ActivationReLU2)


@dataclass
class ExecConfig:  # core.ExecConfig (core/layer.go:147-153)
    Backend: int = BackendCUDA
    MultiCore: bool = True
    TileSize: int = 32


@dataclass(eq=False)
class Layer:  # dense.Layer (layers/dense/dense.go:12-19)
    InputHeight: int
    OutputHeight: int
    Activation: int
    Weights: weights.Store
    Exec: ExecConfig = field(default_factory=ExecConfig)


def NewConfigured(in_: int, out: int, act: int, dt: int, format: quant.Format, init, block_weights: int = 0) -> Layer:
    """dense.NewConfigured (layers/dense/dense.go:47-69)."""
    ws = weights.New(out, in_, init, dt, format, block_weights)
    return Layer(in_, out, act, ws)


def _dims(l: Layer, x: np.ndarray) -> Tuple[int, int, int]:
    if x.ndim < 2:
        raise WelvetError(_lib.WV_ESHAPE, "dense: input shape need [batch,in]")
    batch, in_, out = x.shape[0], l.InputHeight, l.OutputHeight
    if x.shape[1] != in_:
        raise WelvetError(_lib.WV_ESHAPE, f"dense: input width {x.shape[1]} != layer in {in_}")
    if l.Weights.Rows != out or l.Weights.Cols != in_:
        raise WelvetError(_lib.WV_ESHAPE, f"dense: weight shape {l.Weights.Rows}x{l.Weights.Cols} != {out}x{in_}")
    return batch, in_, out


def Activate(v: np.ndarray, act: int) -> np.ndarray:
    """core.Activate (core/activate.go:6-38) over an f64 array. The reference hands an unknown
    activation value back unchanged; here it is an error, so that a layer built with integers
    from another numbering cannot run silently as a linear one."""
    v = np.asarray(v, np.float64)
    if act == ActivationLinear:
        return v
    if act == ActivationReLU:
        return np.where(v < 0, 0.0, v)
    if act == ActivationReLU2:
        return np.where(v < 0, 0.0, v * v)
    if act == ActivationLeakyReLU:
        return np.where(v < 0, 0.01 * v, v)
    if act == ActivationSilu:
        return v / (1.0 + np.exp(-v))
    if act == ActivationGELU:
        return 0.5 * v * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (v + 0.044715 * v * v * v)))
    if act == ActivationTanh:
        return np.tanh(v)
    if act == ActivationSigmoid:
        return 1.0 / (1.0 + np.exp(-v))
    raise WelvetError(_lib.WV_EARG, f"dense: unknown activation {act}")


def MatVecCUDA(s: weights.Store, x: np.ndarray, y: np.ndarray, batch: int, in_: int, out: int) -> None:
    """Twin of dense.MatVecWebGPU (layers/dense/webgpu.go:36-48): y[batch,out] = x[batch,in] W^T."""
    if s is None or s.Packed is None:
        raise WelvetError(_lib.WV_EARG, "dense: nil weights")
    if x.size < batch * in_ or y.size < batch * out:
        raise WelvetError(_lib.WV_ESHAPE, "dense: matvec shape")
    key = quant.EnsureResident(s.Packed)
    xs = np.ascontiguousarray(x.reshape(-1)[: batch * in_], np.float32)
    ys = np.empty(batch * out, np.float32)
    check(lib().wv_matvec(key, xs.ctypes.data, ys.ctypes.data, batch, in_, out))
    y.reshape(-1)[: batch * out] = ys


def MatVecPackedBlob(b: quant.Blob, x: np.ndarray, y: np.ndarray) -> None:
    """dense.MatVecPackedBlob (layers/dense/simd.go:571-614) on the CUDA backend."""
    if b is None:
        raise WelvetError(_lib.WV_EARG, "dense: nil packed blob")
    if x.size < b.Cols or y.size < b.Rows:
        raise WelvetError(_lib.WV_ESHAPE, "dense: packed matvec shape")
    quant.MatVec(b, x, y)


def ForwardCUDA(l: Layer, input: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Shaped like dense.ForwardWebGPU (layers/dense/webgpu.go:17-33): stage x as f32, GEMV on
    the device, then bias + activation (applyBiasAct, dense.go:145-167). Linear / no bias
    aliases post to pre."""
    batch, in_, out = _dims(l, input)
    if l.Activation not in _ACTIVATIONS:
        raise WelvetError(_lib.WV_EARG, f"dense: unknown activation {l.Activation}")
    pre = np.empty((batch, out), input.dtype)
    y = np.empty(batch * out, np.float32)
    MatVecCUDA(l.Weights, np.asarray(input, np.float32), y, batch, in_, out)
    pre[...] = y.reshape(batch, out)
    bias = l.Weights.Bias
    if l.Activation == ActivationLinear and (bias is None or len(bias) == 0):
        return pre, pre
    v = pre.astype(np.float64)
    if bias is not None and len(bias):
        v[:, : len(bias)] += np.asarray(bias, np.float64)[:out]
        pre[...] = v
    with np.errstate(over="ignore"):   # Activate(FromFloat64[T](v), act): v passes through T first (dense.go:163)
        post = Activate(v.astype(input.dtype), l.Activation).astype(input.dtype)
    return pre, post


def Forward(l: Optional[Layer], input: Optional[np.ndarray]) -> Tuple[np.ndarray, np.ndarray]:
    """dense.Forward: dispatch on Exec.Backend. Unknown backends are an error here, not a
    silent CPU route (the reference's own rule, README.md:154)."""
    if l is None or l.Weights is None or input is None:
        raise WelvetError(_lib.WV_EARG, "dense: nil layer/input")
    if l.Exec.Backend == BackendCUDA:
        return ForwardCUDA(l, input)
    raise WelvetError(_lib.WV_EFORMAT, f"dense: backend {l.Exec.Backend} is not provided by welvet_b200 (CUDA only)")


class GatherBuffers:
    """Output vectors for row-sharded GEMVs whose epilogue is the gather (`wv_matvec_dev_gather`):
    one exportable device buffer per rank, every rank's buffer mapped into every process. `exchange`
    takes this rank's 64-byte handle and returns all ranks' handles in rank order (for example
    `torch.distributed.all_gather_object`); with world == 1 it is not called."""

    def __init__(self, nbytes: int, rank: int, world: int, exchange=None):
        import ctypes as C
        L = lib()
        self.rank, self.world, self.nbytes = rank, world, nbytes
        own = C.c_void_p()
        handle = C.create_string_buffer(64)
        check(L.wv_gather_alloc(nbytes, C.byref(own), handle))
        self.own = own.value
        self.ptrs = [None] * world
        self.ptrs[rank] = self.own
        if world > 1:
            handles = exchange(handle.raw)
            for r, h in enumerate(handles):
                if r == rank:
                    continue
                p = C.c_void_p()
                check(L.wv_gather_open(C.create_string_buffer(h, 64), C.byref(p)))
                self.ptrs[r] = p.value
        self._arr = (C.c_void_p * world)(*self.ptrs)

    def pointers(self, offset_floats: int = 0):
        """Array of `world` float pointers, each advanced by offset_floats (one y vector inside the buffers)."""
        import ctypes as C
        return (C.c_void_p * self.world)(*[p + 4 * offset_floats for p in self.ptrs])

    def read(self, offset_floats: int, n: int, rank: Optional[int] = None, stream: int = 0) -> np.ndarray:
        """n floats at offset_floats of rank's buffer (default: this rank's own) as a host array."""
        out = np.empty(n, np.float32)
        check(lib().wv_gather_read(self.ptrs[self.rank if rank is None else rank], 4 * offset_floats, out.ctypes.data, 4 * n, stream))
        return out

    def close_peers(self) -> None:
        """Unmap the other ranks' buffers (every rank does this before any rank frees its own)."""
        for r, p in enumerate(self.ptrs):
            if p is not None and r != self.rank:
                lib().wv_gather_close(p)
                self.ptrs[r] = None

    def free_own(self) -> None:
        if self.ptrs[self.rank] is not None:
            lib().wv_gather_free(self.ptrs[self.rank])
            self.ptrs[self.rank] = None

    def close(self) -> None:
        self.close_peers()
        self.free_own()


def MatVecGatherCUDA(key: int, dx_ptr: int, y_all, world: int, rank: int, row_offset: int, in_: int, out_local: int, stream: int = 0) -> None:
    """Row-sharded y = W x whose kernel stores this rank's rows into every rank's y (no collective)."""
    check(lib().wv_matvec_dev_gather(key, dx_ptr, y_all, world, rank, row_offset, in_, out_local, stream))


def MatVecGroupCUDA(stores, dx_ptr: int, dy_ptrs, batch: int, in_: int, stream: int = 0) -> None:
    """Projection group (Q|K|V, gate|up): y_i = x W_i^T for every store of the list on one shared x, as one
    launch when the stores agree in format and columns (the reference's fused shaders, fusedgpu/shaders.go:59-222).
    Device pointers: dx_ptr to x[batch, in], dy_ptrs[i] to y_i[batch, out_i]."""
    import ctypes as C
    n = len(stores)
    keys = (C.c_uint64 * n)(*[quant.EnsureResident(s.Packed) for s in stores])
    outs = (C.c_int * n)(*[s.Rows for s in stores])
    dys = (C.c_void_p * n)(*dy_ptrs)
    check(lib().wv_matvec_dev_multi(keys, n, dx_ptr, dys, batch, in_, outs, stream))
