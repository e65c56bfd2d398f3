"""ctypes binding of libwelvet_cuda.so (the C ABI declared in include/welvet_cuda.h).

There is no CPU fallback: importing this module without the built library, or calling a
compute entry without a bound sm_100 device, raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# WELVET_CUDA_LIB selects another build of the library (the test-suite loads the variant with the development hooks)
LIB_PATH = os.environ.get("WELVET_CUDA_LIB") or os.path.join(_HERE, "libwelvet_cuda.so")

# Every symbol include/welvet_cuda.h declares.
SYMBOLS = [
    "wv_init", "wv_available", "wv_device_count", "wv_last_error",
    "wv_blob_upload", "wv_blob_upload_wire", "wv_blob_upload_shard", "wv_shard_range",
    "wv_blob_has", "wv_blob_evict", "wv_cache_clear", "wv_cache_bytes", "wv_cache_set_limit",
    "wv_blob_info", "wv_matvec", "wv_matvec_dev", "wv_unpack", "wv_unpack_dev",
    "wv_pack_sizes", "wv_pack", "wv_pack_upload_dev", "wv_device_status", "wv_matvec_dev_static",
    "wv_argmax_dev", "wv_argmax", "wv_matvec_dev_multi", "wv_matvec_dev_gather", "wv_gather_alloc", "wv_gather_open", "wv_gather_close", "wv_gather_free", "wv_gather_read", "wv_gather_signal", "wv_gather_wait", "wv_gather_sync",
    "wv_matvec_dev_swiglu", "wv_matvec_dev_add", "wv_matvec_dev_group_gather", "wv_matvec_dev_fused", "wv_rmsnorm_dev", "wv_rope_cache_dev",
    "wv_attn_decode_dev", "wv_silu_mul_dev", "wv_residual_add_dev",
    "wv_topk_sample_dev", "wv_topk_sample", "wv_decode_row", "wv_decode_row_dev",
]

# Development hooks (csrc/wv_dev_hooks.h): only in a library built with -DWV_DEV_HOOKS (libwelvet_cuda_dev.so),
# for tests and tuning runs; the product library does not export them.
DEV_HOOKS = ["wv_set_tuning", "wv_set_tma_tuning", "wv_set_act_width"]

WV_OK, WV_ESHAPE, WV_EFORMAT, WV_ENOMEM, WV_ECUDA, WV_ETIMEOUT, WV_ENOTFOUND, WV_EINIT, WV_EARG = (
    0, -1, -2, -3, -4, -5, -6, -7, -8)
_NAMES = {-1: "ESHAPE", -2: "EFORMAT", -3: "ENOMEM", -4: "ECUDA", -5: "ETIMEOUT", -6: "ENOTFOUND",
          -7: "EINIT", -8: "EARG"}


class WvFusedCall(C.Structure):
    """WvFusedCall of include/welvet_cuda.h."""
    _fields_ = [("keys", C.POINTER(C.c_uint64)), ("n", C.c_int), ("dx", C.c_void_p), ("y_all", C.POINTER(C.c_void_p)),
                ("world", C.c_int), ("rank", C.c_int), ("row_offset", C.POINTER(C.c_int)), ("in_", C.c_int),
                ("out_local", C.POINTER(C.c_int)), ("mode", C.c_int), ("dresidual", C.c_void_p), ("dnorm_gamma", C.c_void_p),
                ("norm_eps", C.c_double)]


class WelvetError(RuntimeError):
    """A non-zero status from the C ABI (the reference returns Go `error` values)."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"welvet_cuda {_NAMES.get(code, code)}: {msg}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m welvet_b200.build` "
                "(the CUDA backend has no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        u64, i, vp, sz = C.c_uint64, C.c_int, C.c_void_p, C.c_size_t
        L.wv_last_error.restype = C.c_char_p
        L.wv_cache_bytes.restype = u64
        L.wv_cache_clear.restype = None
        L.wv_cache_set_limit.restype = None
        L.wv_cache_set_limit.argtypes = [u64]
        if hasattr(L, "wv_set_tuning"):
            L.wv_set_tuning.restype = None
            L.wv_set_tuning.argtypes = [i, i, i, i]
            L.wv_set_tma_tuning.restype = None
            L.wv_set_tma_tuning.argtypes = [i, i]
            L.wv_set_act_width.restype = None
            L.wv_set_act_width.argtypes = [i]
        L.wv_init.argtypes = [i]
        L.wv_blob_upload.argtypes = [u64, i, i, i, i, i, vp, sz, vp, sz, vp, sz]
        L.wv_blob_upload_wire.argtypes = [u64, i, i, i, i, vp, sz]
        L.wv_blob_upload_shard.argtypes = [u64, i, i, i, i, i, vp, sz, vp, sz, vp, sz, i, i]
        L.wv_shard_range.argtypes = [i, i, i, C.POINTER(i), C.POINTER(i)]
        L.wv_blob_has.argtypes = [u64]
        L.wv_blob_evict.argtypes = [u64]
        L.wv_blob_info.argtypes = [u64, C.POINTER(i), C.POINTER(i), C.POINTER(u64), C.POINTER(u64), C.POINTER(i)]
        L.wv_matvec.argtypes = [u64, vp, vp, i, i, i]
        L.wv_matvec_dev.argtypes = [u64, vp, vp, i, i, i, vp]
        L.wv_matvec_dev_static.argtypes = [u64, vp, vp, i, i, vp]
        L.wv_argmax_dev.argtypes = [vp, i, vp, vp]
        L.wv_argmax.argtypes = [vp, i, C.POINTER(i), vp]
        L.wv_matvec_dev_multi.argtypes = [C.POINTER(u64), i, vp, C.POINTER(vp), i, i, C.POINTER(i), vp]
        L.wv_matvec_dev_gather.argtypes = [u64, vp, C.POINTER(vp), i, i, i, i, i, vp]
        L.wv_gather_alloc.argtypes = [sz, C.POINTER(vp), C.c_char_p]
        L.wv_gather_open.argtypes = [C.c_char_p, C.POINTER(vp)]
        L.wv_gather_close.argtypes = [vp]
        L.wv_gather_free.argtypes = [vp]
        L.wv_gather_signal.argtypes = [C.POINTER(vp), i, i, vp]
        L.wv_gather_wait.argtypes = [vp, i, vp]
        L.wv_gather_sync.argtypes = [C.POINTER(vp), i, i, vp]
        L.wv_gather_read.argtypes = [vp, sz, vp, sz, vp]
        L.wv_matvec_dev_swiglu.argtypes = [u64, u64, vp, vp, i, i, vp]
        L.wv_matvec_dev_add.argtypes = [u64, vp, vp, vp, i, i, vp]
        L.wv_matvec_dev_group_gather.argtypes = [C.POINTER(u64), i, vp, C.POINTER(vp), i, i, C.POINTER(i), i, C.POINTER(i), i, vp, vp]
        L.wv_matvec_dev_fused.argtypes = [C.POINTER(WvFusedCall), vp]
        L.wv_rmsnorm_dev.argtypes = [vp, vp, vp, i, i, C.c_double, vp]
        L.wv_rope_cache_dev.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, C.c_double, vp]
        L.wv_attn_decode_dev.argtypes = [vp, vp, vp, vp, i, i, i, i, i, C.c_float, vp]
        L.wv_silu_mul_dev.argtypes = [vp, vp, vp, i, vp]
        L.wv_residual_add_dev.argtypes = [vp, vp, i, vp]
        L.wv_topk_sample_dev.argtypes = [vp, i, i, C.c_float, i, C.c_double, vp, vp]
        L.wv_topk_sample.argtypes = [vp, i, i, C.c_float, i, C.c_double, C.POINTER(i), vp]
        L.wv_decode_row.argtypes = [u64, i, vp, i]
        L.wv_decode_row_dev.argtypes = [u64, i, vp, vp]
        L.wv_unpack.argtypes = [u64, vp]
        L.wv_unpack_dev.argtypes = [u64, vp, vp]
        L.wv_pack_sizes.argtypes = [i, i, i, i, i, C.POINTER(sz), C.POINTER(sz), C.POINTER(sz)]
        L.wv_pack.argtypes = [i, i, i, vp, i, i, vp, vp, vp]
        L.wv_pack_upload_dev.argtypes = [u64, i, i, i, vp, i, i, vp]
        _lib = L
    return _lib


def has_dev_hooks() -> bool:
    return hasattr(lib(), "wv_set_tuning")


def check(rc: int) -> None:
    if rc != 0:
        raise WelvetError(rc, lib().wv_last_error().decode(errors="replace"))


def init(device: int = -1) -> None:
    """Bind the library to a CUDA device (default: LOCAL_RANK, else 0)."""
    if device < 0:
        device = int(os.environ.get("LOCAL_RANK", "0"))
    check(lib().wv_init(device))
