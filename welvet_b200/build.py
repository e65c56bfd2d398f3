"""In-tree build of libwelvet_cuda.so for sm_100a (nvcc cross-compiles without a GPU).

    python -m welvet_b200.build [--all] [--force] [--verbose]

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
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
# Variants beside the product library: "" is libwelvet_cuda.so (what the package loads); "_dev" adds the development
# hooks of csrc/wv_dev_hooks.h (-DWV_DEV_HOOKS), which the test-suite uses to steer kernel choices. WV_LIB_SUFFIX /
# WV_NVCC_EXTRA build any other variant from the command line.
VARIANTS = {"": [], "_dev": ["-DWV_DEV_HOOKS"]}


def lib_path(suffix: str = "") -> str:
    return os.path.join(HERE, f"libwelvet_cuda{suffix}.so")


LIB = lib_path(os.environ.get("WV_LIB_SUFFIX", ""))

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", INCLUDE]
SOURCES = {
    "wv_layout.cu": ["--fmad=false"],
    "wv_pack.cu": ["--fmad=false"],
    "wv_gemv.cu": [],
    "wv_gemv_tma.cu": [],
    "wv_gemv_mma.cu": [],
    "wv_decode.cu": [],
    "wv_gemv_tc.cu": [],
    "wv_gemm_tcgen05.cu": [],
    "wv_api.cu": [],
}


def _newest_dep() -> float:
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, "welvet_cuda.h"), __file__]
    return max(os.path.getmtime(d) for d in deps)


def _compile(src: str, extra: list[str], objdir: str, verbose: bool) -> str:
    obj = os.path.join(objdir, src.replace(".cu", ".o"))
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


def build(force: bool = False, verbose: bool = False, suffix: str | None = None) -> str:
    """Compile every CUDA source for sm_100a and link one variant of the shared library."""
    if suffix is None:
        suffix = os.environ.get("WV_LIB_SUFFIX", "")
    out = lib_path(suffix)
    if not force and os.path.exists(out) and os.path.getmtime(out) >= _newest_dep():
        return out
    flags = VARIANTS.get(suffix, []) + os.environ.get("WV_NVCC_EXTRA", "").split()
    objdir = os.path.join(HERE, "build" + suffix)
    os.makedirs(objdir, exist_ok=True)
    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda kv: _compile(kv[0], kv[1] + flags, objdir, verbose), SOURCES.items()))
    cmd = ["nvcc", *ARCH, "-shared", "-cudart", "static", "-o", out, *objs]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stderr}")
    return out


def build_all(force: bool = False) -> list[str]:
    """The product library and the development variant the tests load."""
    return [build(force, suffix=s) for s in VARIANTS]


if __name__ == "__main__":
    if "--all" in sys.argv:
        print("\n".join(build_all(force="--force" in sys.argv)))
    else:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
