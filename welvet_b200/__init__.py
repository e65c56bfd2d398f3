"""welvet_b200 — sm_100a backend for Welvet's Dense MatVec (fused dequantise-and-dot GEMV).

Host-side mirror of the reference's quant / weights / layers/dense call surface over the C ABI
of libwelvet_cuda.so. The library must be built (`python -m welvet_b200.build`); there is no
CPU fallback.
"""
from . import _lib, decode, dense, entity, quant, sampling, weights  # noqa: F401
from ._lib import WelvetError, init  # noqa: F401

__all__ = ["quant", "weights", "dense", "decode", "entity", "sampling", "init", "WelvetError"]
