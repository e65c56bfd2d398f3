import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


# The tests load the library variant with the development hooks (kernel-choice steering) when it has been built;
# the product library otherwise, and the tests that steer kernels skip.
_DEV_LIB = os.path.join(ROOT, "welvet_b200", "libwelvet_cuda_dev.so")
if "WELVET_CUDA_LIB" not in os.environ and os.path.exists(_DEV_LIB):
    os.environ["WELVET_CUDA_LIB"] = _DEV_LIB


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100)")


# (oracle name, block_weights, dtype): every layout the backend accepts.
CASES = [(f, 0, 1) for f in [
    "Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K",
    "IQ1_S", "IQ2_XXS", "IQ2_XS", "IQ3_XXS", "IQ3_S", "IQ4_NL", "IQ4_XS",
    "TernaryPacked", "BinaryPacked", "AffinePacked"]] + [
    ("BinaryPacked", 128, 1), ("none", 0, 1), ("none", 0, 2), ("none", 0, 3)]


def case_id(c):
    f, bw, dt = c
    if f == "none":
        return {1: "f32", 2: "f16", 3: "bf16"}[dt]
    return f + ("_g128" if bw == 128 else "")


def case_ok(c, rows, cols):
    f, bw, _ = c
    if f == "AffinePacked":
        return cols % 64 == 0
    if bw == 128:
        return cols % 128 == 0
    return True


def make_w(seed, rows, cols, sigma=0.02):
    rng = np.random.default_rng(seed)
    w = rng.normal(0, sigma, (rows, cols)).astype(np.float32)
    x = rng.normal(0, 1, cols).astype(np.float32)
    return w, x


@pytest.fixture(scope="session")
def wv():
    """The product package bound to cuda:0 (GPU tests only)."""
    import welvet_b200
    welvet_b200.init(0)
    return welvet_b200


@pytest.fixture
def hooks(wv):
    """The development hooks of the loaded library; skips where it was built without them."""
    if not wv._lib.has_dev_hooks():
        pytest.skip("library built without -DWV_DEV_HOOKS")
    return wv._lib.lib()


def to_product_blob(wvpkg, ob):
    """oracle.Blob -> welvet_b200.quant.Blob (same arrays, reference field names)."""
    q = wvpkg.quant
    return q.Blob(q.Format(ob.format), ob.rows, ob.cols, ob.raw.copy(), ob.scales.copy(), ob.mins.copy(),
                  ob.block_weights, ob.dtype)
