"""Host-side mirror of the reference's token pickers (model/sampling/argmax.go:4-18, topk.go:11-50) on the
device: the LM head's logits stay in HBM and only the index comes back."""
from __future__ import annotations

import ctypes as C
import random

from ._lib import check, lib


def ArgMaxCUDA(d_logits: int, n: int, stream: int = 0) -> int:
    """sampling.ArgMax over n device floats at address d_logits (first strict maximum; NaN never wins)."""
    idx = C.c_int()
    check(lib().wv_argmax(d_logits, n, C.byref(idx), stream))
    return idx.value


def SampleTopKCUDA(d_logits: int, n: int, topK: int, temperature: float, deterministic: bool = False,
                   u: float | None = None, stream: int = 0) -> int:
    """sampling.SampleTopK over n device floats. `u` is the uniform draw the reference takes from math/rand inside
    the call (random.random() when omitted). At most 1024 candidates on the device."""
    idx = C.c_int()
    if u is None:
        u = random.random()
    check(lib().wv_topk_sample(d_logits, n, topK, temperature, 1 if deterministic else 0, u, C.byref(idx), stream))
    return idx.value
