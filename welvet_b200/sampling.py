"""Host-side mirror of the reference's greedy pick (model/sampling/argmax.go:4-18) on the device:
the LM head's logits stay in HBM and only the index comes back."""
from __future__ import annotations

import ctypes as C

from ._lib import check, lib


def ArgMaxCUDA(d_logits: int, n: int, stream: int = 0) -> int:
    """sampling.ArgMax over n device floats at address d_logits (first strict maximum; NaN never wins)."""
    idx = C.c_int()
    check(lib().wv_argmax(d_logits, n, C.byref(idx), stream))
    return idx.value
