"""In-tree build of libwelvet_cuda.so for sm_100a (nvcc cross-compiles without a GPU).

    python -m welvet_b200.build [--force] [--verbose]

wv_layout.cu and wv_pack.cu hold the bit-exact arithmetic (unpack / pack) and are compiled
with --fmad=false so that no multiply-add is contracted; the GEMV may use FMA.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build" + os.environ.get("WV_LIB_SUFFIX", ""))
# WV_LIB_SUFFIX builds a second library beside the product one (development variants, e.g. with -DWV_PHASES)
_SUFFIX = os.environ.get("WV_LIB_SUFFIX", "")
LIB = os.path.join(HERE, f"libwelvet_cuda{_SUFFIX}.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", INCLUDE] + os.environ.get("WV_NVCC_EXTRA", "").split()
SOURCES = {
    "wv_layout.cu": ["--fmad=false"],
    "wv_pack.cu": ["--fmad=false"],
    "wv_gemv.cu": [],
    "wv_gemv_tma.cu": [],
    "wv_gemv_mma.cu": [],
    "wv_decode.cu": [],
    "wv_gemv_tc.cu": [],
    "wv_api.cu": [],
}


def _newest_dep() -> float:
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, "welvet_cuda.h"), __file__]
    return max(os.path.getmtime(d) for d in deps)


def _compile(src: str, extra: list[str], verbose: bool) -> str:
    obj = os.path.join(OBJ, src.replace(".cu", ".o"))
    cmd = ["nvcc", *ARCH, *COMMON, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stderr}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a and link the shared library."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_dep():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda kv: _compile(kv[0], kv[1], verbose), SOURCES.items()))
    cmd = ["nvcc", *ARCH, "-shared", "-cudart", "static", "-o", LIB, *objs]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
