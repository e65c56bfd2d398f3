"""Generates tests/golden/golden_small.npz: packed bytes, dequantised weights and reference
outputs for every layout on two small seeded shapes.

    python tests/golden/make_golden.py

The reference (Go) cannot run where this was written, so the vectors come from the CPU oracle
after it has been checked against the second numpy restatement and the hand-derived
known-answer blocks in tests/test_oracle.py. They pin the CUDA path and guard the oracle
against regressions.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))
import oracle as O  # noqa: E402
from conftest import CASES, case_id, case_ok  # noqa: E402

SHAPES = [(8, 512), (3, 100)]


def main():
    out = {}
    for rows, cols in SHAPES:
        rng = np.random.default_rng(1000 + rows * cols)
        w = rng.normal(0, 0.02, (rows, cols)).astype(np.float32)
        x = rng.normal(0, 1, cols).astype(np.float32)
        out[f"w_{rows}x{cols}"] = w
        out[f"x_{rows}x{cols}"] = x
        for c in CASES:
            if not case_ok(c, rows, cols):
                continue
            f, bw, dt = c
            b = O.pack(f, w, rows, cols, bw, dt)
            k = f"{case_id(c)}_{rows}x{cols}"
            out[k + "_raw"] = b.raw
            out[k + "_scales"] = b.scales
            out[k + "_mins"] = b.mins
            out[k + "_unpack"] = O.unpack(b)
            out[k + "_y_scalar"] = O.matvec(b, x)
            if cols % 32 == 0:
                out[k + "_y_simd"] = O.matvec_simd(b, x, 1)
    np.savez_compressed(os.path.join(HERE, "golden_small.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
