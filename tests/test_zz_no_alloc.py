"""The allocation-free GEMV entry (wv_matvec_dev_static) against the regular device entry.

Collected last on purpose: a run that stops at the first failure has then already run every
other test. The entry exists for embedders that cannot allocate device memory any more when
they call in (all of HBM already committed to their own pools, or a decode loop that must not
take cudaMalloc's device-wide synchronisation); it keeps the activation scratch in a fixed
array inside the library. Two calls in a row must both match wv_matvec_dev within the
output tolerance the other GPU tests use (1e-3 * sum|w x| per row): the second call runs on
the scratch contents the first one left behind."""
import numpy as np
import pytest

import oracle as O
from conftest import make_w

pytestmark = pytest.mark.gpu
TOL = 1e-3


@pytest.mark.parametrize("fmt,bw", [("Q4_K", 0), ("Q8_0", 0), ("Q5_1", 0), ("IQ3_S", 0), ("BinaryPacked", 128), ("AffinePacked", 64)])
def test_static_scratch_entry_matches_regular_entry(wv, fmt, bw):
    import torch
    from welvet_b200 import _lib
    L = _lib.lib()
    rows, cols = 203, 4096
    w, x1 = make_w(77, rows, cols)
    x2 = np.random.default_rng(78).normal(0, 3, cols).astype(np.float32)
    ob = O.pack(fmt, w, rows, cols, bw)
    key = 0x2A0000 + ob.format
    _lib.check(L.wv_blob_upload(key, ob.format, 1, rows, cols, ob.block_weights, ob.raw.ctypes.data, ob.raw.size,
                                ob.scales.ctypes.data if ob.scales.size else None, ob.scales.size,
                                ob.mins.ctypes.data if ob.mins.size else None, ob.mins.size))
    try:
        for x in (x1, x2):  # two calls in a row share the static scratch
            dx = torch.from_numpy(x).cuda()
            y_ref = torch.zeros(rows, device="cuda")
            y_new = torch.full((rows,), float("nan"), device="cuda")
            _lib.check(L.wv_matvec_dev(key, dx.data_ptr(), y_ref.data_ptr(), 1, cols, rows, None))
            _lib.check(L.wv_matvec_dev_static(key, dx.data_ptr(), y_new.data_ptr(), cols, rows, None))
            torch.cuda.synchronize()
            assert L.wv_device_status() == 0
            den = O.sum_abs_wx(ob, x)
            err = np.abs(y_new.cpu().numpy().astype(np.float64) - y_ref.cpu().numpy().astype(np.float64))
            assert np.all(err <= TOL * den + 1e-30), f"worst {np.max(err / np.maximum(den, 1e-30)):.3e}"
            # and against the oracle itself
            ref = O.matvec_simd(ob, x, 1)
            assert np.all(np.abs(y_new.cpu().numpy().astype(np.float64) - ref) <= TOL * den + 1e-30)
    finally:
        L.wv_blob_evict(key)


def test_static_scratch_entry_rejects_what_it_cannot_do(wv):
    import torch
    from welvet_b200 import _lib
    L = _lib.lib()
    x = torch.zeros(40000, device="cuda")
    y = torch.zeros(64, device="cuda")
    # beyond the static maximum of 32768 columns
    rows, cols = 4, 33792
    w, _ = make_w(1, rows, cols)
    ob = O.pack("Q4_0", w, rows, cols)
    _lib.check(L.wv_blob_upload(0x2B0001, ob.format, 1, rows, cols, 32, ob.raw.ctypes.data, ob.raw.size, None, 0, None, 0))
    assert L.wv_matvec_dev_static(0x2B0001, x.data_ptr(), y.data_ptr(), cols, rows, None) == _lib.WV_ESHAPE
    assert b"exceeds the static scratch maximum" in L.wv_last_error()
    L.wv_blob_evict(0x2B0001)
    # a format whose kernel has no scratch
    ob = O.pack("IQ4_NL", w[:, :1024], rows, 1024)
    _lib.check(L.wv_blob_upload(0x2B0002, ob.format, 1, rows, 1024, 32, ob.raw.ctypes.data, ob.raw.size, ob.scales.ctypes.data, ob.scales.size, None, 0))
    assert L.wv_matvec_dev_static(0x2B0002, x.data_ptr(), y.data_ptr(), 1024, rows, None) == _lib.WV_EFORMAT
    assert L.wv_matvec_dev_static(0x2B0002, x.data_ptr(), y.data_ptr(), 512, rows, None) == _lib.WV_ESHAPE
    L.wv_blob_evict(0x2B0002)
    assert L.wv_matvec_dev_static(0x2B0003, x.data_ptr(), y.data_ptr(), 1024, rows, None) == _lib.WV_ENOTFOUND


def test_static_scratch_entry_at_its_maximum_width_from_another_thread_without_allocating(wv):
    """The widest shape the fixed array takes (32768 columns: the whole array and the kernel's largest
    shared-memory record), called from a host thread that has never touched CUDA (such a thread starts
    with device 0 current, whatever device the library is bound to), with the device's free memory
    compared before and after a warmed call: the entry must not allocate."""
    import threading
    import torch
    from welvet_b200 import _lib
    L = _lib.lib()
    rows, cols = 37, 32768
    w, x = make_w(79, rows, cols)
    ob = O.pack("Q4_K", w, rows, cols)
    key = 0x2C0001
    _lib.check(L.wv_blob_upload(key, ob.format, 1, rows, cols, 0, ob.raw.ctypes.data, ob.raw.size, None, 0, None, 0))
    try:
        dx = torch.from_numpy(x).cuda()
        y = torch.full((rows,), float("nan"), device="cuda")
        _lib.check(L.wv_matvec_dev_static(key, dx.data_ptr(), y.data_ptr(), cols, rows, None))   # first call: set-up
        torch.cuda.synchronize()
        result = {}

        def worker():
            free0, _ = torch.cuda.mem_get_info()
            result["rc"] = L.wv_matvec_dev_static(key, dx.data_ptr(), y.data_ptr(), cols, rows, None)
            torch.cuda.synchronize()
            free1, _ = torch.cuda.mem_get_info()
            result["delta"] = free0 - free1
        t = threading.Thread(target=worker)
        t.start()
        t.join()
        assert result["rc"] == 0, L.wv_last_error()
        assert result["delta"] == 0, f"free device memory changed by {result['delta']} bytes across the call"
        assert L.wv_device_status() == 0
        den = O.sum_abs_wx(ob, x)
        ref = O.matvec_simd(ob, x, 1)
        assert np.all(np.abs(y.cpu().numpy().astype(np.float64) - ref) <= TOL * den + 1e-30)
    finally:
        L.wv_blob_evict(key)
