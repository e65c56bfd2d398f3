"""Writes tests/golden/ref_inputs.bin: the seeded inputs the Go program oracle/ref_dump/main.go feeds to
the reference's own Pack / Unpack / MatVec. Seeds 0-5 (the seeds of the benchmark configs), every
packed format plus FormatNone f32, small shapes including a ragged one and a matrix with zero blocks.

    python tests/golden/make_ref_inputs.py

Format of the file (little endian): u32 ncases, then per case u32 format | u32 rows | u32 cols |
f32 w[rows*cols] | f32 x[cols]. numpy's default_rng is the canonical generator (the reference
defines none for this path)."""
import os
import struct

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SHAPES = [(8, 512), (3, 100), (16, 256), (5, 4096)]
FORMATS = list(range(0, 21))   # quant.Format values (quant/format.go:9-39)


def cases():
    for seed in range(6):
        rows, cols = SHAPES[seed % len(SHAPES)]
        rng = np.random.default_rng(seed)
        w = rng.normal(0, 0.02, (rows, cols)).astype(np.float32)
        x = rng.normal(0, 1, cols).astype(np.float32)
        if rows >= 8:
            w[1, :64] = 0.0
            w[2, :] = 0.0
        for f in FORMATS:
            if f == 20 and cols % 64:      # AffinePacked g64 needs whole groups per row
                continue
            yield f, rows, cols, w, x


def main():
    cs = list(cases())
    path = os.path.join(HERE, "ref_inputs.bin")
    with open(path, "wb") as fh:
        fh.write(struct.pack("<I", len(cs)))
        for f, rows, cols, w, x in cs:
            fh.write(struct.pack("<III", f, rows, cols))
            fh.write(w.astype("<f4").tobytes())
            fh.write(x.astype("<f4").tobytes())
    print(path, len(cs), "cases", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
