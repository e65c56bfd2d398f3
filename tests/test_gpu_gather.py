"""Row-sharded GEMV whose epilogue is the gather (`wv_matvec_dev_gather`). On one GPU two ranks are
emulated with two output buffers of the same process: each shard's launch must leave its rows in
BOTH buffers, and the assembled vectors must equal the unsharded result bit for bit. Covers the
dp4a bulk-copy kernel, the tensor-pipe kernel and the paths that finish with a copy kernel
(FormatNone, ragged columns). With two visible GPUs a second test runs two processes whose buffers
are mapped into each other through the library's IPC plumbing."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import oracle as O
from conftest import make_w

pytestmark = pytest.mark.gpu
CASES = [("Q4_K", 0, 1, 256, 4096), ("Q4_0", 0, 1, 256, 4096), ("Q8_0", 0, 1, 96, 14336), ("Q6_K", 0, 1, 200, 1024),
         ("IQ4_NL", 0, 1, 64, 4096), ("none", 0, 1, 64, 2048), ("none", 0, 3, 64, 2048), ("Q5_1", 0, 1, 40, 96),
         ("BinaryPacked", 128, 1, 128, 4096), ("AffinePacked", 64, 1, 128, 4096)]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"{c[0]}{c[1] or ''}_dt{c[2]}_{c[3]}x{c[4]}")
def test_gather_epilogue_two_emulated_ranks(wv, case):
    f, bw, dt, rows, cols = case
    L = wv._lib.lib()
    w, x = make_w(21, rows, cols)
    ob = O.pack(f, w, rows, cols, bw, dt)
    args = (O.FMT[f], dt, rows, cols, ob.block_weights, ob.raw.ctypes.data, ob.raw.size,
            ob.scales.ctypes.data if ob.scales.size else None, ob.scales.size, ob.mins.ctypes.data if ob.mins.size else None, ob.mins.size)
    world = 2
    keys = [0xA10000 + r for r in range(world)]
    full = 0xA1FFFF
    bufs = [wv.dense.GatherBuffers(4 * rows, 0, 1) for _ in range(world)]
    try:
        wv._lib.check(L.wv_blob_upload(full, *args))
        for r in range(world):
            wv._lib.check(L.wv_blob_upload_shard(keys[r], *args, r, world))
        dx = torch.from_numpy(x).cuda()
        ref = torch.zeros(rows, device="cuda")
        wv._lib.check(L.wv_matvec_dev(full, dx.data_ptr(), ref.data_ptr(), 1, cols, rows, None))
        y_all = (C.c_void_p * world)(*[b.own for b in bufs])
        for r in range(world):
            r0, r1 = C.c_int(), C.c_int()
            wv._lib.check(L.wv_shard_range(rows, r, world, C.byref(r0), C.byref(r1)))
            wv._lib.check(L.wv_matvec_dev_gather(keys[r], dx.data_ptr(), y_all, world, r, r0.value, cols, r1.value - r0.value, None))
        torch.cuda.synchronize()
        want = ref.cpu().numpy()
        for b in bufs:
            got = b.read(0, rows)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    finally:
        for k in keys + [full]:
            L.wv_blob_evict(k)
        for b in bufs:
            b.close()


def test_arrival_flags_in_stream_order_and_timeout(wv):
    """Two emulated ranks on one stream: both signal, then both waits pass at once (nothing on one GPU ever waits
    for work queued behind it). A wait that nobody signals runs out, is reported through wv_device_status and
    leaves the context usable."""
    L = wv._lib.lib()
    world = 2
    flags = [wv.dense.GatherBuffers(4 * (world + 2), 0, 1) for _ in range(world)]
    try:
        f_all = (C.c_void_p * world)(*[f.own for f in flags])
        for step in range(1, 4):
            for r in range(world):
                wv._lib.check(L.wv_gather_signal(f_all, world, r, None))
            for r in range(world):
                wv._lib.check(L.wv_gather_wait(flags[r].own, world, None))
            torch.cuda.synchronize()
            assert L.wv_device_status() == 0
            for r in range(world):
                words = flags[r].read(0, world + 2).view(np.uint32)
                assert list(words) == [step, step, step, step]
        # rank 0 waits for a step that rank 1 never signals
        wv._lib.check(L.wv_gather_signal(f_all, world, 0, None))
        wv._lib.check(L.wv_gather_wait(flags[0].own, world, None))
        torch.cuda.synchronize()
        assert L.wv_device_status() == wv._lib.WV_ETIMEOUT
        assert L.wv_device_status() == 0                      # reported once
        y = torch.arange(8, dtype=torch.float32, device="cuda")
        assert wv.sampling.ArgMaxCUDA(y.data_ptr(), 8) == 7   # the context still works
    finally:
        for f in flags:
            f.close()


def test_signal_and_wait_in_one_launch(wv):
    """wv_gather_sync: the signal and the wait of a step as one kernel. Alone on its own flags it passes at once;
    with a second emulated rank whose signal is already in the stream it passes too, and leaves the same counters
    as the two separate launches."""
    L = wv._lib.lib()
    one = wv.dense.GatherBuffers(4 * 3, 0, 1)
    try:
        f1 = (C.c_void_p * 1)(one.own)
        for step in range(1, 4):
            wv._lib.check(L.wv_gather_sync(f1, 1, 0, None))
            torch.cuda.synchronize()
            assert L.wv_device_status() == 0
            assert list(one.read(0, 3).view(np.uint32)) == [step, step, step]
    finally:
        one.close()
    world = 2
    flags = [wv.dense.GatherBuffers(4 * (world + 2), 0, 1) for _ in range(world)]
    try:
        f_all = (C.c_void_p * world)(*[f.own for f in flags])
        for step in range(1, 3):
            wv._lib.check(L.wv_gather_signal(f_all, world, 1, None))     # rank 1's rows are in
            wv._lib.check(L.wv_gather_sync(f_all, world, 0, None))       # rank 0 signals and finds both words there
            wv._lib.check(L.wv_gather_wait(flags[1].own, world, None))
            torch.cuda.synchronize()
            assert L.wv_device_status() == 0
            for r in range(world):
                assert list(flags[r].read(0, world + 2).view(np.uint32)) == [step] * 4
        assert L.wv_gather_sync(f_all, 9, 0, None) == wv._lib.WV_EARG
    finally:
        for f in flags:
            f.close()


def test_gather_argument_errors(wv):
    L = wv._lib.lib()
    y_all = (C.c_void_p * 1)(0)
    assert L.wv_matvec_dev_gather(1, None, y_all, 1, 0, 0, 32, 1, None) == wv._lib.WV_EARG
    dx = torch.zeros(32, device="cuda")
    assert L.wv_matvec_dev_gather(0xDEAD, dx.data_ptr(), y_all, 9, 0, 0, 32, 1, None) == wv._lib.WV_EARG      # more than 8 ranks
    assert L.wv_matvec_dev_gather(0xDEAD, dx.data_ptr(), y_all, 1, 0, 0, 32, 1, None) == wv._lib.WV_ENOTFOUND


CHILD = r"""
import os, sys, ctypes as C
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import welvet_b200 as wv, oracle as O
from conftest import make_w
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank); wv.init(rank)
dist.init_process_group("gloo")
L = wv._lib.lib()
def exchange(h):
    out = [None] * world
    dist.all_gather_object(out, h)
    return out
rows, cols = 512, 4096
bufs = wv.dense.GatherBuffers(4 * rows * 3, rank, world, exchange)
ok = True
for slot, f in enumerate(["Q4_K", "Q4_0", "Q8_0"]):
    w, x = make_w(30 + slot, rows, cols)
    ob = O.pack(f, w, rows, cols)
    args = (O.FMT[f], 1, rows, cols, ob.block_weights, ob.raw.ctypes.data, ob.raw.size, None, 0, None, 0)
    wv._lib.check(L.wv_blob_upload_shard(100 + slot, *args, rank, world))
    wv._lib.check(L.wv_blob_upload(200 + slot, *args))
    r0, r1 = C.c_int(), C.c_int()
    L.wv_shard_range(rows, rank, world, C.byref(r0), C.byref(r1))
    dx = torch.from_numpy(x).cuda()
    ref = torch.zeros(rows, device="cuda")
    wv._lib.check(L.wv_matvec_dev(200 + slot, dx.data_ptr(), ref.data_ptr(), 1, cols, rows, None))
    wv._lib.check(L.wv_matvec_dev_gather(100 + slot, dx.data_ptr(), bufs.pointers(slot * rows), world, rank, r0.value, cols, r1.value - r0.value, None))
    torch.cuda.synchronize()
    dist.barrier()                      # every rank's kernel has finished: all slices are in place
    got = bufs.read(slot * rows, rows)
    ok = ok and np.array_equal(got.view(np.uint32), ref.cpu().numpy().view(np.uint32))
# chained steps ordered by arrival flags only: gather GEMV -> signal -> wait -> pick over the whole gathered vector
flags = wv.dense.GatherBuffers(4 * (world + 2), rank, world, exchange)
f_all = (C.c_void_p * world)(*flags.ptrs)
picks = torch.zeros(6, dtype=torch.int32, device="cuda")
refs = []
for step in range(6):
    slot = step % 3
    x = np.random.default_rng(100 + step).normal(0, 1, cols).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    ref = torch.zeros(rows, device="cuda")
    wv._lib.check(L.wv_matvec_dev(200 + slot, dx.data_ptr(), ref.data_ptr(), 1, cols, rows, None))
    refs.append(int(torch.argmax(ref).item()))
    L.wv_shard_range(rows, rank, world, C.byref(r0), C.byref(r1))
    wv._lib.check(L.wv_matvec_dev_gather(100 + slot, dx.data_ptr(), bufs.pointers(slot * rows), world, rank, r0.value, cols, r1.value - r0.value, None))
    wv._lib.check(L.wv_gather_signal(f_all, world, rank, None))
    wv._lib.check(L.wv_gather_wait(flags.own, world, None))
    wv._lib.check(L.wv_argmax_dev(bufs.own + 4 * slot * rows, rows, picks.data_ptr() + 4 * step, None))
torch.cuda.synchronize()
ok = ok and L.wv_device_status() == 0 and picks.cpu().tolist() == refs
dist.barrier()
flags.close_peers(); bufs.close_peers()
dist.barrier()
flags.free_own(); bufs.free_own()
dist.destroy_process_group()
print("RANK", rank, "OK" if ok else "MISMATCH")
sys.exit(0 if ok else 1)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_gather_two_processes_two_gpus(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29533")
        procs.append(subprocess.Popen([sys.executable, str(script), root], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
