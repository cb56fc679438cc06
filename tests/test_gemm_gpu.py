"""GPU parity of the matmul node against the CPU oracle, through the C ABI.

Tolerances: bf16 operands / fp32 accumulate / bf16 output within max-abs 2e-2 of the
oracle's fp32 result on the same bf16-rounded inputs (entries are N(0,1)/sqrt(K), so
outputs are O(1)); fp32 path within max-rel 1e-4.
"""
import numpy as np
import pytest

import habu_b200 as hb
import oracle
from util import SEED, bf16_close, bf16_normal, max_abs, max_rel

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def run_bf16(ctx, M, N, K, a_mn=False, b_mn=False, config_id=-1, epilogue=hb.HB_EPI_NONE):
    A, Ab = bf16_normal((M, K), SEED + 1, K ** -0.5)
    Bt, Btb = bf16_normal((N, K), SEED + 2, 1.0)   # B column-major == Bt row-major
    dA = ctx.upload(np.ascontiguousarray(Ab.T)).T if a_mn else ctx.upload(Ab)
    dB = ctx.upload(np.ascontiguousarray(Btb.T)) if b_mn else ctx.upload(Btb).T
    R = Rb = dR = None
    if epilogue == hb.HB_EPI_RESIDUAL:
        R, Rb = bf16_normal((M, N), SEED + 3)
        dR = ctx.upload(Rb)
    dC = ctx.matmul(dA, dB, epilogue=epilogue, residual=dR, config_id=config_id)
    ctx.sync()
    got = oracle.from_bf16_bits(ctx.download(dC))
    ref = oracle.gemm(A, Bt.T)
    if epilogue == hb.HB_EPI_GELU:
        ref = oracle.gelu(ref)
    elif epilogue == hb.HB_EPI_SWIGLU:
        ref = oracle.swiglu(ref, interleaved=True)
    elif epilogue == hb.HB_EPI_RESIDUAL:
        ref = ref + R
    for t in (dA, dB, dC) + ((dR,) if dR else ()):
        ctx.free(t)
    return got, ref


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 512), (1024, 1024, 1024)])
def test_bf16_square_and_small(ctx, M, N, K):
    got, ref = run_bf16(ctx, M, N, K)
    assert max_abs(got, ref) < TOL_BF16


@pytest.mark.parametrize("M,N,K", [(16, 512, 1024), (1, 8, 8), (130, 264, 72), (300, 1000, 520), (129, 257 * 8, 64)])
def test_bf16_ragged_shapes(ctx, M, N, K):
    got, ref = run_bf16(ctx, M, N, K)
    assert max_abs(got, ref) < TOL_BF16


@pytest.mark.parametrize("M,N,K", [(16, 8192, 8192), (1, 256, 512), (7, 1000, 1096), (33, 4096, 2048), (64, 384, 8192)])
def test_bf16_skinny_split_k_path(ctx, M, N, K):
    # M <= 64 takes the swapped-operand split-K kernel; its slice-ordered reduction is
    # deterministic, so two runs agree bit for bit
    got, ref = run_bf16(ctx, M, N, K)
    assert max_abs(got, ref) < TOL_BF16
    again, _ = run_bf16(ctx, M, N, K)
    assert np.array_equal(got, again)
    forced, _ = run_bf16(ctx, M, N, K, config_id=4)      # the general kernel on the same shape
    assert max_abs(forced, ref) < TOL_BF16


def test_bf16_every_config(ctx):
    for i, cfg in enumerate(hb.matmul_configs()):
        got, ref = run_bf16(ctx, 384, 768, 320, config_id=i)
        assert max_abs(got, ref) < TOL_BF16, (i, cfg.tile_n, cfg.stages)


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
def test_bf16_mn_major_operands(ctx, a_mn, b_mn):
    got, ref = run_bf16(ctx, 256, 384, 192, a_mn=a_mn, b_mn=b_mn)
    assert max_abs(got, ref) < TOL_BF16
    got, ref = run_bf16(ctx, 200, 136, 72, a_mn=a_mn, b_mn=b_mn)
    assert max_abs(got, ref) < TOL_BF16
    # every configuration (one-CTA tiles and CTA-pair tiles) on a ragged multi-tile shape
    for i in range(len(hb.matmul_configs())):
        got, ref = run_bf16(ctx, 520, 776, 200, a_mn=a_mn, b_mn=b_mn, config_id=i)
        assert max_abs(got, ref) < TOL_BF16, i


@pytest.mark.parametrize("epi", [hb.HB_EPI_GELU, hb.HB_EPI_SWIGLU, hb.HB_EPI_RESIDUAL])
def test_bf16_epilogues(ctx, epi):
    # epilogue outputs reach |x| ~ 10, where one bf16 rounding alone exceeds 2e-2
    got, ref = run_bf16(ctx, 256, 512, 256, epilogue=epi)
    assert bf16_close(got, ref) < 0
    got, ref = run_bf16(ctx, 100, 200, 64, epilogue=epi)
    assert bf16_close(got, ref) < 0


def test_bf16_many_tiles_persistent_schedule(ctx):
    # more tiles than SMs: every CTA walks several tiles and both accumulators
    got, ref = run_bf16(ctx, 2048, 4096, 256)
    assert max_abs(got, ref) < TOL_BF16


def test_bf16_linearity_property_full_size(ctx):
    # 8192^3 is too slow for the oracle; check C(A, B) rows against a row sample computed
    # on the CPU, and that the host-buffer entry point agrees with the device one.
    M = N = K = 8192
    A, Ab = bf16_normal((M, K), SEED + 11, K ** -0.5)
    Bt, Btb = bf16_normal((N, K), SEED + 12)
    dA, dB = ctx.upload(Ab), ctx.upload(Btb)
    dC = ctx.matmul(dA, dB.T)
    ctx.sync()
    got = oracle.from_bf16_bits(ctx.download(dC))
    rows = np.array([0, 1, 127, 128, 4095, 4097, 8191])
    ref = oracle.gemm(np.ascontiguousarray(A[rows]), Bt.T)
    assert max_abs(got[rows], ref) < TOL_BF16
    cols = np.array([0, 255, 256, 5000, 8191])
    ref_c = oracle.gemm(A, np.ascontiguousarray(Bt[cols]).T)
    assert max_abs(got[:, cols], ref_c) < TOL_BF16
    host = oracle.from_bf16_bits(ctx.matmul_host(Ab, Btb))
    assert np.array_equal(host, got)
    for t in (dA, dB, dC):
        ctx.free(t)


def test_host_entry_point_pipelines_row_chunks(ctx):
    # M >= 2048 goes through the host call as four to eight row chunks over the copy-in, compute and
    # copy-out streams; two calls in a row reuse the staging buffer and the events
    M, N, K = 2048, 264, 136
    A, Ab = bf16_normal((M, K), SEED + 15, K ** -0.5)
    Bt, Btb = bf16_normal((N, K), SEED + 16)
    ref = oracle.gemm(A, Bt.T)
    for _ in range(2):
        host = oracle.from_bf16_bits(ctx.matmul_host(Ab, Btb))
        assert max_abs(host, ref) < TOL_BF16


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (100, 37, 50), (1, 1, 1)])
def test_f32_path(ctx, M, N, K):
    A = oracle.uniform((M, K), SEED + 21)
    B = oracle.uniform((K, N), SEED + 22)
    ref = oracle.gemm(A, B, acc_double=True)
    dA, dB = ctx.upload(A), ctx.upload(B)
    got = ctx.download(ctx.matmul(dA, dB))
    assert max_rel(got, ref) < 1e-4
    # column-major B through the host entry point
    got2 = ctx.matmul_host(A, np.ascontiguousarray(B.T), dtype=hb.HB_F32)
    assert max_rel(got2, ref) < 1e-4


def test_invalid_arguments_are_reported_not_launched(ctx):
    a = ctx.empty((64, 64))
    b = ctx.empty((32, 64))
    with pytest.raises(hb.HabuError) as e:
        ctx.matmul(a, b.T.T)           # inner dimensions differ
    assert e.value.status == 1
    c = ctx.empty((64, 60))            # K = 60 row pitch is not a multiple of 8
    with pytest.raises(hb.HabuError) as e:
        ctx.matmul(c, ctx.wrap(b.ptr, (60, 32), stride=(1, 60)))
    assert e.value.status == 7
    with pytest.raises(hb.HabuError):
        ctx.matmul(a, a.T, config_id=999)
    ctx.sync()


def test_gathered_entry_point_is_the_plain_matmul_on_one_rank(ctx):
    """hb_matmul_gathered waits for rows that a fused collective on other ranks publishes; with a
    single rank there is nothing to wait for and it must be the plain matmul, bit for bit."""
    import ctypes as C
    from habu_b200 import _capi, model_ir
    M, N, K = 512, 384, 256
    A, Ab = bf16_normal((M, K), SEED + 900, K ** -0.5)
    B, Bb = bf16_normal((N, K), SEED + 901)
    dA, dB = ctx.upload(Ab), ctx.upload(Bb)
    want = ctx.download(ctx.matmul(dA, dB.T))
    out = ctx.empty((M, N))
    ta, tb, tc = dA.c(), dB.T.c(), out.c()
    opts = _capi.hb_matmul_opts(hb.HB_EPI_NONE, -1, None, 0)
    ctx._check(model_ir._lib.hb_matmul_gathered(ctx._h, C.byref(ta), C.byref(tb), C.byref(tc), C.byref(opts)))
    ctx.sync()
    assert np.array_equal(ctx.download(out), want)
    assert max_abs(oracle.from_bf16_bits(want), oracle.gemm(A, B.T)) < TOL_BF16


def test_comm_configure_validates_its_arguments(ctx):
    ctx.comm_configure(1, 0)
    ctx.comm_configure(2, 64)
    ctx.comm_configure(0, 0)
    for bad in ((3, 0), (-1, 0), (1, -5)):
        with pytest.raises(hb.HabuError) as e:
            ctx.comm_configure(*bad)
        assert e.value.status == 1


def test_weight_matrix_promise_changes_the_launch_not_the_result(ctx):
    """HB_MATMUL_WEIGHTS_B lets the M <= 64 kernel stream B in before the kernel in front of it on
    the stream has finished; a chain of such products (each reading the previous one's output as
    its A, the situation of a generation step) must give the bits of the plainly ordered chain."""
    M, K = 16, 1024
    A, Ab = bf16_normal((M, K), SEED + 910, K ** -0.5)
    Ws = [bf16_normal((K, K), SEED + 911 + i, K ** -0.5) for i in range(4)]
    dWs = [ctx.upload(wb) for _, wb in Ws]
    outs = []
    for weights in (False, True):
        x = ctx.upload(Ab)
        for dW in dWs * 3:                      # twelve dependent products back to back
            x = ctx.matmul(x, dW.T, weights=weights)
        ctx.sync()
        outs.append(ctx.download(x))
    assert np.array_equal(outs[0], outs[1])
    ref = A
    for W, _ in Ws * 3:
        ref = oracle.round_bf16(oracle.gemm(ref, W.T))
    assert bf16_close(oracle.from_bf16_bits(outs[1]), ref) < 0
