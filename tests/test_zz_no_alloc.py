"""The allocation-free skinny matmul (``hb_matmul_skinny_static``).

Some callers cannot allocate device memory at the moment they need a product: a serving
loop that forbids allocator locks and the device-wide synchronisation an allocation or a
free can trigger, or a foreign-runtime callback that must not block in the driver.  For
them the library keeps the split-K scratch in a static device array.  This test calls
that entry point through the C ABI twice in a row and checks both results against the
ordinary matmul node (same kernel, context-owned scratch): within the bf16 tolerance of
the other matmul tests, and -- because the slice-ordered reduction is deterministic --
bit for bit.  The second call must also leave the amount of free device memory exactly as
it found it (the property the entry point exists for: nothing is allocated, nothing
freed).  It also checks that an over-size problem is refused with a message, and that a
device index that is not the calling thread's current device is refused.

Collected last on purpose, so a run that stops at the first failure has already run
every other test.
"""
import ctypes as C

import numpy as np
import pytest

import oracle
from util import SEED, bf16_normal, max_abs

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def _free_device_bytes():
    import torch
    free, _ = torch.cuda.mem_get_info(0)
    return free


def _static(lib, dA, dB, dC, M, N, K):
    st = lib.hb_matmul_skinny_static(C.c_void_p(dA.ptr), C.c_void_p(dB.ptr), C.c_void_p(dC.ptr), M, N, K, 0, None)
    assert st == 0, lib.hb_static_last_error().decode()
    words = (C.c_int32 * 4)()
    assert lib.hb_static_status(0, words) == 0      # blocks until the default stream drains
    assert words[0] == 0, list(words)


@pytest.mark.parametrize("M,N,K", [(16, 8192, 8192), (5, 1024, 4096)])
def test_static_scratch_matches_the_matmul_node_twice_in_a_row(ctx, M, N, K):
    from habu_b200 import model_ir
    lib = model_ir._lib
    A, Ab = bf16_normal((M, K), SEED + 91, K ** -0.5)
    Bt, Btb = bf16_normal((N, K), SEED + 92)
    dA, dB = ctx.upload(Ab), ctx.upload(Btb)
    want = ctx.download(ctx.matmul(dA, dB.T))
    ref = oracle.gemm(A, Bt.T)
    assert max_abs(oracle.from_bf16_bits(want), ref) < TOL_BF16
    dC = ctx.empty((M, N))
    zeros = np.zeros((M, N), np.uint16)
    for call in range(2):
        ctx._check(model_ir._lib.hb_upload(ctx._h, dC.ptr, zeros.ctypes.data_as(C.c_void_p), M * N * 2))
        ctx.sync()
        before = _free_device_bytes()
        _static(lib, dA, dB, dC, M, N, K)
        if call == 1:     # the first call on a device may load the kernel image; the second allocates nothing
            assert _free_device_bytes() == before, "the allocation-free call changed the free device memory"
        got = ctx.download(dC)
        assert max_abs(oracle.from_bf16_bits(got), ref) < TOL_BF16, call
        assert np.array_equal(got, want), call
    for t in (dA, dB, dC):
        ctx.free(t)


def test_static_scratch_refuses_problems_beyond_its_size(ctx):
    from habu_b200 import model_ir
    lib = model_ir._lib
    d = ctx.empty((8,))
    # refused before anything is launched, so the tiny buffer is never touched:
    # 64 x 16384 x 65536 needs 128 tiles x 3 K-ranges x 128 x 64 partial floats, over the 2^20 limit
    st = lib.hb_matmul_skinny_static(C.c_void_p(d.ptr), C.c_void_p(d.ptr), C.c_void_p(d.ptr), 64, 16384, 65536, 0, None)
    assert st == 7
    assert b"exceeds the static scratch" in lib.hb_static_last_error()
    # more than 1024 column tiles
    st = lib.hb_matmul_skinny_static(C.c_void_p(d.ptr), C.c_void_p(d.ptr), C.c_void_p(d.ptr), 16, 128 * 1025, 1024, 0, None)
    assert st == 7 and b"exceeds the static scratch" in lib.hb_static_last_error()
    st = lib.hb_matmul_skinny_static(C.c_void_p(d.ptr), C.c_void_p(d.ptr), C.c_void_p(d.ptr), 65, 1024, 1024, 0, None)
    assert st == 7 and b"at most 64" in lib.hb_static_last_error()
    # a device that is not the calling thread's current one is refused by both entry points
    # (the static arrays' addresses are looked up on the current device)
    words = (C.c_int32 * 4)()
    assert lib.hb_static_status(63, words) == 1 and b"current CUDA device" in lib.hb_static_last_error()
    st = lib.hb_matmul_skinny_static(C.c_void_p(d.ptr), C.c_void_p(d.ptr), C.c_void_p(d.ptr), 16, 1024, 1024, 63, None)
    assert st == 1 and b"current CUDA device" in lib.hb_static_last_error()
    ctx.free(d)
