"""Model-IR executor: node validation, the lifetime-based memory planner and the
two-stream launcher, on small graphs checked against the oracle."""
import numpy as np
import pytest

import habu_b200 as hb
import oracle
from habu_b200.graph import Graph
from util import SEED, bf16_close, bf16_normal

pytestmark = pytest.mark.gpu


def test_unknown_tensor_and_read_before_write_are_errors(ctx):
    g = Graph(ctx)
    a = g.temp((64, 64))
    with pytest.raises(hb.HabuError) as e:
        g.gelu(99, a)
    assert e.value.status == 2                      # `Not_found
    b = g.temp((64, 64))
    g.gelu(a, b)                                    # reads planner-owned `a` that nothing wrote
    with pytest.raises(hb.HabuError) as e:
        g.plan()
    assert e.value.status == 1 and "before any node writes it" in str(e.value)
    with pytest.raises(hb.HabuError):
        g.run()                                     # not planned
    g.close()


def test_planner_reuses_dead_tensors_and_results_match_oracle(ctx):
    rows, cols = 256, 512
    x, xb = bf16_normal((rows, cols), SEED + 101)
    dx = ctx.upload(xb)
    dout = ctx.empty((rows, cols))
    g = Graph(ctx)
    i, o = g.input(dx), g.input(dout)
    t = [g.temp((rows, cols)) for _ in range(6)]
    g.gelu(i, t[0])
    for k in range(5):
        g.gelu(t[k], t[k + 1])                      # a chain: at most two temporaries are ever live
    g.add(t[5], i, o)
    arena, sym = g.plan()
    assert sym == 0 and arena <= 2 * rows * cols * 2 + 512
    text = g.describe()
    assert text.count("gelu") == 6 and "arena+0" in text
    g.run()
    ctx.sync()
    ref = x
    for _ in range(6):
        ref = oracle.round_bf16(oracle.gelu(ref))
    assert bf16_close(oracle.from_bf16_bits(ctx.download(dout)), ref + x) < 0
    g.close()


def test_views_and_matmul_attention_nodes(ctx):
    B, S, H, D = 1, 256, 2, 128
    W = 3 * H * D
    x, xb = bf16_normal((B * S, 256), SEED + 102)
    w, wb = bf16_normal((W, 256), SEED + 103, 256 ** -0.5)
    g = Graph(ctx)
    xi, wi = g.input(ctx.upload(xb)), g.input(ctx.upload(wb).T)
    qkv = g.temp((B * S, W))
    g.matmul(xi, wi, qkv)
    v4 = lambda off: g.view(qkv, off, (B, S, H, D), (S * W, W, D, 1))
    dout = ctx.empty((B, S, H, D))
    g.attention(v4(0), v4(H * D), v4(2 * H * D), g.input(dout))
    g.plan()
    g.run()
    ctx.sync()
    full = oracle.round_bf16(oracle.gemm(x, w.T)).reshape(B, S, 3, H, D)
    ref = oracle.attention(np.ascontiguousarray(full[:, :, 0]), np.ascontiguousarray(full[:, :, 1]),
                           np.ascontiguousarray(full[:, :, 2]))
    assert bf16_close(oracle.from_bf16_bits(ctx.download(dout)), ref) < 0
    g.close()


def test_side_stream_nodes_are_ordered_by_their_data(ctx):
    # all_reduce on one rank is the identity, but it still travels on the side stream, so
    # the event dependencies between the two streams are exercised: producer -> collective
    # -> consumer, repeated, with memory reuse in between.
    n = 1 << 20
    x, xb = bf16_normal((n,), SEED + 104)
    dx, dout = ctx.upload(xb), ctx.empty((n,))
    g = Graph(ctx)
    i, o = g.input(dx), g.input(dout)
    cur = i
    for k in range(4):
        a = g.temp((n,), symmetric=True)
        g.gelu(cur, a)
        g.all_reduce(a, stream=1)
        b = g.temp((n,))
        g.add(a, i, b)
        cur = b
    g.add(cur, i, o)
    g.plan()
    for _ in range(3):
        g.run()
    ctx.sync()
    ref = x
    for k in range(4):
        ref = oracle.round_bf16(oracle.round_bf16(oracle.gelu(ref)) + x)
    ref = ref + x
    assert bf16_close(oracle.from_bf16_bits(ctx.download(dout)), ref) < 0
    g.close()


def test_view_past_the_end_of_a_planner_tensor_is_rejected(ctx):
    g = Graph(ctx)
    t = g.temp((16, 64))
    ok = g.view(t, 64, (15, 64), (64, 1))
    assert ok >= 0
    with pytest.raises(hb.HabuError) as e:
        g.view(t, 64, (16, 64), (64, 1))            # one row too many
    assert e.value.status == 1
    with pytest.raises(hb.HabuError):
        g.view(ok, 64 * 14, (2, 64), (64, 1))       # nested view: offsets accumulate
    g.close()
