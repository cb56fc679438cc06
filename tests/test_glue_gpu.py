"""GPU parity of the glue operators against the CPU oracle, through the C ABI.
bf16 outputs are compared with the oracle's fp32 result on the same bf16-rounded inputs:
max-abs 2e-2 widened by one bf16 output rounding; gathers and argmax are bit-exact."""
import numpy as np
import pytest

import habu_b200 as hb
import oracle
from util import SEED, bf16_close, bf16_normal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(7, 64), (33, 4096), (5, 8192), (2, 16384)])
def test_rmsnorm(ctx, rows, cols):
    x, xb = bf16_normal((rows, cols), SEED + 61)
    g, gb = bf16_normal((cols,), SEED + 62, 0.3)
    g += 1.0
    g = oracle.round_bf16(g)
    gb = oracle.to_bf16_bits(g)
    got = oracle.from_bf16_bits(ctx.download(ctx.rmsnorm(ctx.upload(xb), ctx.upload(gb), eps=1e-5)))
    assert bf16_close(got, oracle.rmsnorm(x, g, 1e-5)) < 0


def test_rmsnorm_with_fused_residual_add(ctx):
    rows, cols = 19, 4096
    x, xb = bf16_normal((rows, cols), SEED + 63)
    r, rb = bf16_normal((rows, cols), SEED + 64)
    g = np.ones(cols, np.float32)
    dR = ctx.upload(rb)
    dY = ctx.rmsnorm(ctx.upload(xb), ctx.upload(oracle.to_bf16_bits(g)), residual=dR)
    new_r = oracle.round_bf16(x + r)
    assert np.array_equal(oracle.from_bf16_bits(ctx.download(dR)), new_r)
    assert bf16_close(oracle.from_bf16_bits(ctx.download(dY)), oracle.rmsnorm(new_r, g, 1e-5)) < 0


@pytest.mark.parametrize("tokens,seq,heads,hd,pos0", [(8, 8, 2, 128, 0), (64, 16, 5, 128, 0), (4096, 2048, 3, 128, 0), (6, 3, 1, 64, 100)])
def test_rope(ctx, tokens, seq, heads, hd, pos0):
    x, xb = bf16_normal((tokens, heads * hd), SEED + 65)
    d = ctx.upload(xb)
    ctx.rope(d, seq=seq, heads=heads, head_dim=hd, pos0=pos0)
    got = oracle.from_bf16_bits(ctx.download(d))
    assert bf16_close(got, oracle.rope(x, seq, heads, hd, 10000.0, pos0)) < 0


def test_rope_on_a_strided_slice_leaves_the_rest_untouched(ctx):
    tokens, W, heads, hd = 32, 6 * 128, 4, 128      # rotate the first 4 of 6 heads per row
    x, xb = bf16_normal((tokens, W), SEED + 66)
    d = ctx.upload(xb)
    ctx.rope(ctx.wrap(d.ptr, (tokens, heads * hd), stride=(W, 1)), seq=32, heads=heads, head_dim=hd)
    got = oracle.from_bf16_bits(ctx.download(d))
    ref = x.copy()
    ref[:, :heads * hd] = oracle.rope(np.ascontiguousarray(x[:, :heads * hd]), 32, heads, hd)
    assert np.array_equal(got[:, heads * hd:], x[:, heads * hd:])
    assert bf16_close(got, ref) < 0


def test_embedding_is_a_bit_exact_gather(ctx):
    table, tb = bf16_normal((1000, 256), SEED + 67)
    ids = (np.arange(333) * 7919 % 1000).astype(np.int32)
    got = ctx.download(ctx.embedding(ctx.upload(tb), ctx.upload(ids)))
    assert np.array_equal(got, tb[ids])


def test_embedding_out_of_range_id_is_reported(ctx):
    table, tb = bf16_normal((10, 64), SEED + 68)
    ids = np.array([1, 10, 2], np.int32)
    out = ctx.embedding(ctx.upload(tb), ctx.upload(ids))
    with pytest.raises(hb.HabuError) as e:
        ctx.sync()
    assert e.value.status == 1
    got = ctx.download(out)
    assert np.array_equal(got[0], tb[1]) and not got[1].any()


@pytest.mark.parametrize("rows,half", [(3, 8), (100, 1792), (17, 14336)])
def test_swiglu(ctx, rows, half):
    x, xb = bf16_normal((rows, 2 * half), SEED + 69)
    got = oracle.from_bf16_bits(ctx.download(ctx.swiglu(ctx.upload(xb))))
    assert bf16_close(got, oracle.swiglu(x)) < 0


@pytest.mark.parametrize("n", [1, 7, 8, 1000, 1 << 20])
def test_gelu_add_and_gelu_backward(ctx, n):
    x, xb = bf16_normal((n,), SEED + 70, 2.0)
    y, yb = bf16_normal((n,), SEED + 71)
    dx, dy = ctx.upload(xb), ctx.upload(yb)
    assert bf16_close(oracle.from_bf16_bits(ctx.download(ctx.gelu(dx))), oracle.gelu(x)) < 0
    assert bf16_close(oracle.from_bf16_bits(ctx.download(ctx.add(dx, dy))), x + y) < 0
    assert bf16_close(oracle.from_bf16_bits(ctx.download(ctx.gelu_backward(dx, dy))), oracle.gelu_backward(x, y)) < 0


def test_argmax_is_bit_exact_and_first_index_wins(ctx):
    x, xb = bf16_normal((37, 5000), SEED + 72)
    got = ctx.download(ctx.argmax(ctx.upload(xb)))
    assert np.array_equal(got, oracle.argmax(x))
    tie = np.zeros((3, 777), np.float32)
    tie[1, 5] = tie[1, 600] = 2.0
    tie[2, 776] = 1.0
    got = ctx.download(ctx.argmax(ctx.upload(oracle.to_bf16_bits(tie))))
    assert list(got) == [0, 5, 776]
