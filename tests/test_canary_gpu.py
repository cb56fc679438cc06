"""Out-of-bounds writes, checked without a memory checker: every operator writes its output
into the middle of a larger device buffer filled with a pattern (guard bands in front and
behind, padding columns at the end of every row where the operator takes a row pitch, a start
that is not 16-byte aligned where the operator allows it).  After the call the pattern must be
intact everywhere outside the output, and the output must still match the oracle, so a store
that strays by one element on a ragged edge shows up as a failed test instead of as silent
corruption of a neighbouring tensor.
"""
import numpy as np
import pytest

import habu_b200 as hb
import oracle
from util import SEED, bf16_close, bf16_normal, max_abs, max_rel

pytestmark = pytest.mark.gpu

GUARD = 4096            # pattern elements in front of and behind the output
_PAT = {hb.HB_BF16: (np.uint16, 0xBEEF), hb.HB_F32: (np.uint32, 0xBEEFBEEF), hb.HB_I32: (np.uint32, 0x7EEFBEEF)}


class Guarded:
    """A [rows, cols] output view (row pitch cols + row_pad, start shifted by `shift` elements)
    inside a pattern-filled device buffer."""

    def __init__(self, ctx, rows, cols, dtype=hb.HB_BF16, row_pad=0, shift=0, shape=None):
        self.ctx, self.rows, self.cols, self.ld, self.dtype = ctx, rows, cols, cols + row_pad, dtype
        self.np_dtype, self.pat = _PAT[dtype]
        self.front = GUARD + shift
        self.total = self.front + rows * self.ld + GUARD
        host = np.full(self.total, self.pat, self.np_dtype)
        up = host if dtype == hb.HB_BF16 else host.view(np.float32 if dtype == hb.HB_F32 else np.int32)
        self.buf = ctx.upload(up)
        ptr = self.buf.ptr + self.front * host.itemsize
        if shape is None:
            self.t = ctx.wrap(ptr, (rows, cols), dtype, (self.ld, 1), owner=self.buf)
        else:                                   # contiguous N-d output of rows * cols elements
            assert row_pad == 0
            self.t = ctx.wrap(ptr, shape, dtype, owner=self.buf)

    def finish(self):
        """Downloads the buffer, asserts the pattern outside the output, returns the output."""
        self.ctx.sync()
        raw = self.ctx.download(self.buf).view(self.np_dtype)
        body = raw[self.front:self.front + self.rows * self.ld].reshape(self.rows, self.ld)
        assert (raw[:self.front] == self.pat).all(), "write in front of the output"
        assert (raw[self.front + self.rows * self.ld:] == self.pat).all(), "write behind the output"
        assert (body[:, self.cols:] == self.pat).all(), "write into the padding between rows"
        self.ctx.free(self.buf)
        out = np.ascontiguousarray(body[:, :self.cols])
        return out if self.dtype == hb.HB_BF16 else out.view(np.float32 if self.dtype == hb.HB_F32 else np.int32)


# ragged edges in every dimension; (row_pad, shift): aligned and packed, aligned with padded rows,
# odd pitch and a start that is not 16-byte aligned (the scalar store path)
@pytest.mark.parametrize("row_pad,shift", [(0, 0), (8, 0), (3, 1)])
@pytest.mark.parametrize("M,N,K", [(130, 264, 72), (300, 1000, 520), (513, 776, 136), (7, 1000, 1096), (33, 264, 520)])
def test_matmul_stays_inside_its_output(ctx, M, N, K, row_pad, shift):
    A, Ab = bf16_normal((M, K), SEED + 1, K ** -0.5)
    Bt, Btb = bf16_normal((N, K), SEED + 2)
    dA, dB = ctx.upload(Ab), ctx.upload(Btb)
    g = Guarded(ctx, M, N, row_pad=row_pad, shift=shift)
    ctx.matmul(dA, dB.T, out=g.t)
    got = oracle.from_bf16_bits(g.finish())
    assert max_abs(got, oracle.gemm(A, Bt.T)) < 2e-2
    ctx.free(dA), ctx.free(dB)


@pytest.mark.parametrize("cluster,tile_n", [(1, 256), (1, 128), (1, 64), (2, 256), (2, 128)])
def test_every_tile_shape_stays_inside_its_output(ctx, cluster, tile_n):
    # one configuration of each tile shape forced, on a shape whose last tile is ragged in M and N
    M, N, K = 300, 1000, 520
    cfg = next(c.config_id for c in hb.matmul_configs() if c.cluster == cluster and c.tile_n == tile_n)
    A, Ab = bf16_normal((M, K), SEED + 3, K ** -0.5)
    Bt, Btb = bf16_normal((N, K), SEED + 4)
    dA, dB = ctx.upload(Ab), ctx.upload(Btb)
    g = Guarded(ctx, M, N, row_pad=8)
    ctx.matmul(dA, dB.T, out=g.t, config_id=cfg)
    got = oracle.from_bf16_bits(g.finish())
    assert max_abs(got, oracle.gemm(A, Bt.T)) < 2e-2
    ctx.free(dA), ctx.free(dB)


@pytest.mark.parametrize("epi", [hb.HB_EPI_GELU, hb.HB_EPI_SWIGLU, hb.HB_EPI_RESIDUAL])
def test_matmul_epilogues_stay_inside_their_output(ctx, epi):
    M, N, K = 130, 528, 72
    A, Ab = bf16_normal((M, K), SEED + 5, K ** -0.5)
    Bt, Btb = bf16_normal((N, K), SEED + 6)
    R, Rb = bf16_normal((M, N), SEED + 7)
    dA, dB, dR = ctx.upload(Ab), ctx.upload(Btb), ctx.upload(Rb)
    g = Guarded(ctx, M, N // 2 if epi == hb.HB_EPI_SWIGLU else N, row_pad=8)
    ctx.matmul(dA, dB.T, out=g.t, epilogue=epi, residual=dR if epi == hb.HB_EPI_RESIDUAL else None)
    got = oracle.from_bf16_bits(g.finish())
    ref = oracle.gemm(A, Bt.T)
    ref = {hb.HB_EPI_GELU: oracle.gelu, hb.HB_EPI_SWIGLU: lambda x: oracle.swiglu(x, interleaved=True),
           hb.HB_EPI_RESIDUAL: lambda x: x + R}[epi](ref)
    assert bf16_close(got, ref) < 0
    for t in (dA, dB, dR):
        ctx.free(t)


@pytest.mark.parametrize("M,N,K", [(100, 37, 50), (33, 65, 17)])
def test_f32_matmul_stays_inside_its_output(ctx, M, N, K):
    A = oracle.uniform((M, K), SEED + 8)
    B = oracle.uniform((K, N), SEED + 9)
    dA, dB = ctx.upload(A), ctx.upload(np.ascontiguousarray(B.T))
    g = Guarded(ctx, M, N, dtype=hb.HB_F32, row_pad=3, shift=1)
    ctx.matmul(dA, dB.T, out=g.t)
    assert max_rel(g.finish(), oracle.gemm(A, B)) < 1e-4
    ctx.free(dA), ctx.free(dB)


@pytest.mark.parametrize("S,causal", [(200, True), (129, True), (333, False)])
def test_attention_stays_inside_its_output(ctx, S, causal):
    # ragged sequence lengths: the last query tile and the last key tile are partial
    B, Hq, Hkv, D = 2, 4, 2, 128
    Q, Qb = bf16_normal((B, S, Hq, D), SEED + 10)
    K, Kb = bf16_normal((B, S, Hkv, D), SEED + 11)
    V, Vb = bf16_normal((B, S, Hkv, D), SEED + 12)
    dQ, dK, dV = ctx.upload(Qb), ctx.upload(Kb), ctx.upload(Vb)
    g = Guarded(ctx, B * S, Hq * D, shape=(B, S, Hq, D))
    gl = Guarded(ctx, B * Hq, S, dtype=hb.HB_F32, shape=(B, Hq, S))
    ctx.attention(dQ, dK, dV, out=g.t, causal=causal, lse=gl.t)
    got = oracle.from_bf16_bits(g.finish()).reshape(B, S, Hq, D)
    lse = gl.finish().reshape(B, Hq, S)
    ref, ref_lse = oracle.attention(Q, K, V, causal=causal, return_lse=True)
    assert max_abs(got, ref) < 2e-2
    assert max_abs(lse, ref_lse) < 1e-2
    for t in (dQ, dK, dV):
        ctx.free(t)


@pytest.mark.parametrize("B,length,hint", [(3, 1, 0), (5, 77, 0), (16, 300, 300), (2, 511, 0)])
def test_decode_operators_stay_inside_their_outputs(ctx, B, length, hint):
    # the cache append may touch one position of every sequence and nothing else; the single-query
    # attention (several key ranges per sequence, merged by the last one to finish) only its output
    Hq, Hkv, D, s_max = 8, 2, 128, 512
    W = (Hq + 2 * Hkv) * D
    pos = length - 1
    _, qkv_b = bf16_normal((B, W), SEED + 13)
    _, cache_b = bf16_normal((2 * B, s_max, Hkv, D), SEED + 14)
    gk = Guarded(ctx, 2 * B * s_max, Hkv * D, shape=(2 * B, s_max, Hkv, D))
    ctx._check(hb.model_ir._lib.hb_upload(ctx._h, gk.t.ptr, cache_b.ctypes.data, cache_b.nbytes))
    d_qkv = ctx.upload(qkv_b)
    d_pos = ctx.upload(np.full(1, pos, np.int32))
    ctx.rope_append(d_qkv, gk.t, d_pos, Hq, Hkv)
    go = Guarded(ctx, B, Hq * D, row_pad=0)
    ctx.attention_decode(d_qkv, gk.t, d_pos, Hq, Hkv, out=go.t, len_hint=hint)
    out = oracle.from_bf16_bits(go.finish())
    rotated = ctx.download(d_qkv)
    cache = gk.finish().reshape(2 * B, s_max, Hkv, D)
    # only position `pos` of every sequence changed, to the rotated k and the v of the new token
    want = cache_b.copy()
    want[:B, pos] = rotated[:, Hq * D:(Hq + Hkv) * D].reshape(B, Hkv, D)
    want[B:, pos] = qkv_b[:, (Hq + Hkv) * D:].reshape(B, Hkv, D)
    assert np.array_equal(cache, want)
    # and the attention output is the softmax over positions 0..pos of that cache
    q = oracle.from_bf16_bits(rotated[:, :Hq * D]).reshape(B, Hq, D)
    Kc = oracle.from_bf16_bits(cache[:B, :length]).astype(np.float64)
    Vc = oracle.from_bf16_bits(cache[B:, :length]).astype(np.float64)
    ref = np.empty((B, Hq, D))
    for h in range(Hq):
        s = np.einsum("bd,bld->bl", q[:, h].astype(np.float64), Kc[:, :, h // (Hq // Hkv)]) * D ** -0.5
        p = np.exp(s - s.max(-1, keepdims=True))
        ref[:, h] = np.einsum("bl,bld->bd", p / p.sum(-1, keepdims=True), Vc[:, :, h // (Hq // Hkv)])
    assert max_abs(out, ref.reshape(B, Hq * D)) < 2e-2
    ctx.free(d_qkv), ctx.free(d_pos)


@pytest.mark.parametrize("rows,cols", [(37, 512), (1, 4096), (130, 1040), (5, 272)])
def test_glue_operators_stay_inside_their_outputs(ctx, rows, cols):
    X, Xb = bf16_normal((rows, cols), SEED + 15)
    Y, Yb = bf16_normal((rows, cols), SEED + 16)
    G, Gb = bf16_normal((cols,), SEED + 17)
    dX, dY, dG = ctx.upload(Xb), ctx.upload(Yb), ctx.upload(Gb)
    f = oracle.from_bf16_bits

    g = Guarded(ctx, rows, cols)
    ctx.rmsnorm(dX, dG, out=g.t)
    assert bf16_close(f(g.finish()), oracle.rmsnorm(X, G)) < 0

    g = Guarded(ctx, rows, cols)
    ctx.rmsnorm(dX, dG, out=g.t, residual=dY)                 # dY becomes X + Y, the output its norm
    assert bf16_close(f(g.finish()), oracle.rmsnorm(oracle.round_bf16(X + Y), G)) < 0
    ctx._check(hb.model_ir._lib.hb_upload(ctx._h, dY.ptr, Yb.ctypes.data, Yb.nbytes))
    ctx.sync()

    g = Guarded(ctx, rows, cols)
    ctx.add(dX, dY, out=g.t)
    assert bf16_close(f(g.finish()), X + Y) < 0

    g = Guarded(ctx, rows, cols)
    ctx.gelu(dX, out=g.t)
    assert bf16_close(f(g.finish()), oracle.gelu(X)) < 0

    g = Guarded(ctx, rows, cols)
    ctx.gelu_backward(dX, dY, out=g.t)
    assert bf16_close(f(g.finish()), oracle.gelu_backward(X, Y)) < 0

    g = Guarded(ctx, rows, cols // 2)
    ctx.swiglu(dX, out=g.t)
    assert bf16_close(f(g.finish()), oracle.swiglu(X)) < 0

    for t in (dX, dY, dG):
        ctx.free(t)


def test_gather_and_argmax_stay_inside_their_outputs(ctx):
    vocab, dim, tokens = 101, 264, 53
    _, Tb = bf16_normal((vocab, dim), SEED + 18)
    ids = (np.arange(tokens, dtype=np.int32) * 7) % vocab
    dT, dI = ctx.upload(Tb), ctx.upload(ids)
    g = Guarded(ctx, tokens, dim)
    ctx.embedding(dT, dI, out=g.t)
    assert np.array_equal(g.finish(), Tb[ids])
    ctx.free(dT), ctx.free(dI)
