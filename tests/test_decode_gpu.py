"""Decode-shaped path: RoPE + cache append, split-KV single-query attention, and the whole
generation step through the executor.

Parity: the attention kernel against a float64 numpy evaluation of the same cache (max-abs
2e-2, bf16 output); the appended cache rows against the oracle's RoPE (one bf16 rounding); the
step graph token by token against (a) the oracle's decode_step in bf16-storage mode and (b) the
device's own prefill graph over the same tokens -- token t of the decode path must equal row t
of the prefill path within the bf16 tolerance, although the two share no kernel but RMSNorm."""
import ctypes as C

import numpy as np
import pytest

import oracle
from habu_b200.tp import DecoderConfig, DecodeGraph, DecoderGraph, decode_layer, shard_layer
from oracle import decoder
from util import SEED, bf16_close, bf16_normal, max_abs

pytestmark = pytest.mark.gpu


def _up(ctx, t, a):
    from habu_b200 import model_ir
    a = np.ascontiguousarray(a)
    ctx._check(model_ir._lib.hb_upload(ctx._h, C.c_void_p(t.ptr), a.ctypes.data_as(C.c_void_p), a.nbytes))
    ctx.sync()


def _ref_attention(q, K, V, L):
    """q [B,Hq,D], K/V [B,S,Hkv,D] -> [B,Hq*D] in float64 over positions < L."""
    B, Hq, D = q.shape
    Hkv = K.shape[2]
    qh = q.reshape(B, Hkv, Hq // Hkv, D).astype(np.float64)
    s = np.einsum("bkgd,blkd->bkgl", qh, K[:, :L].astype(np.float64)) / np.sqrt(D)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    return np.einsum("bkgl,blkd->bkgd", p, V[:, :L].astype(np.float64)).reshape(B, Hq * D)


@pytest.mark.parametrize("B,Hq,Hkv,s_max,lengths,hint", [
    (2, 8, 2, 300, [1, 63, 64, 65, 300], 0),          # ragged lengths around the 64-position tile
    (16, 32, 8, 2048, [2048, 1000], 0),               # the benchmark's shape: 4 query heads per KV head
    (1, 8, 1, 4096, [4096, 3], 0),                    # one sequence, 8 query heads on one KV head, many splits
    (3, 4, 4, 700, [700, 129], 128),                  # no grouping; a length hint far below the true length
])
def test_split_kv_attention_matches_numpy(ctx, B, Hq, Hkv, s_max, lengths, hint):
    D = 128
    W = (Hq + 2 * Hkv) * D
    qkv, qkv_b = bf16_normal((B, W), SEED + 700)
    K, Kb = bf16_normal((B, s_max, Hkv, D), SEED + 701)
    V, Vb = bf16_normal((B, s_max, Hkv, D), SEED + 702)
    d_qkv = ctx.upload(qkv_b)
    d_kv = ctx.upload(np.concatenate([Kb, Vb], 0))
    d_pos = ctx.upload(np.zeros(1, np.int32))
    q = qkv[:, :Hq * D].reshape(B, Hq, D)
    for L in lengths:
        _up(ctx, d_pos, np.array([L - 1], np.int32))
        out1 = ctx.download(ctx.attention_decode(d_qkv, d_kv, d_pos, Hq, Hkv, len_hint=hint))
        out2 = ctx.download(ctx.attention_decode(d_qkv, d_kv, d_pos, Hq, Hkv, len_hint=hint))
        assert np.array_equal(out1, out2), "the split merge must not depend on scheduling"
        assert max_abs(oracle.from_bf16_bits(out1), _ref_attention(q, K, V, L)) < 2e-2, L
    for t in (d_qkv, d_kv, d_pos):
        ctx.free(t)


def test_rope_append_writes_the_rotated_token_and_refuses_a_full_cache(ctx):
    from habu_b200.model_ir import HabuError
    B, Hq, Hkv, D, s_max = 3, 4, 2, 128, 40
    W = (Hq + 2 * Hkv) * D
    qkv, qkv_b = bf16_normal((B, W), SEED + 710)
    d_kv = ctx.upload(np.zeros((2 * B, s_max, Hkv, D), np.uint16))
    d_pos = ctx.upload(np.zeros(1, np.int32))
    for pos in (0, 7, 39):
        d_qkv = ctx.upload(qkv_b)
        _up(ctx, d_pos, np.array([pos], np.int32))
        ctx.rope_append(d_qkv, d_kv, d_pos, Hq, Hkv)
        ctx.sync()
        got = oracle.from_bf16_bits(ctx.download(d_qkv))
        want_q = oracle.rope(np.ascontiguousarray(qkv[:, :Hq * D]), 1, Hq, D, pos0=pos)
        want_k = oracle.rope(np.ascontiguousarray(qkv[:, Hq * D:(Hq + Hkv) * D]), 1, Hkv, D, pos0=pos)
        tol = lambda ref: 2.0 ** -8 * np.maximum(np.abs(ref), 1.0)
        assert np.all(np.abs(got[:, :Hq * D] - want_q) <= tol(want_q))
        assert np.all(np.abs(got[:, Hq * D:(Hq + Hkv) * D] - want_k) <= tol(want_k))
        assert np.array_equal(got[:, (Hq + Hkv) * D:], qkv[:, (Hq + Hkv) * D:])        # values untouched
        cache = ctx.download(d_kv)
        assert np.array_equal(cache[:B, pos].reshape(B, -1), ctx.download(d_qkv)[:, Hq * D:(Hq + Hkv) * D])
        assert np.array_equal(cache[B:, pos].reshape(B, -1), qkv_b[:, (Hq + Hkv) * D:])
        ctx.free(d_qkv)
    # a full cache: nothing is written, the next sync reports it, and the context stays usable
    before = ctx.download(d_kv)
    d_qkv = ctx.upload(qkv_b)
    _up(ctx, d_pos, np.array([s_max], np.int32))
    ctx.rope_append(d_qkv, d_kv, d_pos, Hq, Hkv)
    with pytest.raises(HabuError) as err:
        ctx.sync()
    assert err.value.status == 1 and "kernel tag 5" in str(err.value)
    assert np.array_equal(ctx.download(d_kv), before)
    ctx.advance_pos(d_pos, -s_max)
    ctx.sync()
    assert int(ctx.download(d_pos)[0]) == 0


def test_generation_steps_match_the_oracle_and_the_prefill_path(ctx):
    S = 40
    cfg = DecoderConfig(d_model=512, n_q_heads=4, n_kv_heads=2, head_dim=128, ffn_hidden=1024, n_layers=2, batch=2, seq=S)
    layers = [decoder.make_layer(cfg, i) for i in range(cfg.n_layers)]
    x0 = decoder.make_input(cfg)                                    # [batch * S, d]
    bits = lambda lw: {k: oracle.to_bf16_bits(v) for k, v in lw.items()}
    # the device's prefill path over the same tokens
    pre = DecoderGraph(ctx, cfg, 1, 0, [bits(shard_layer(l, cfg, 1, 0)) for l in layers])
    pre.plan()
    _up(ctx, pre.x0, oracle.to_bf16_bits(x0))
    pre.run()
    ctx.sync()
    prefill = oracle.from_bf16_bits(ctx.download(pre.out)).reshape(cfg.batch, S, -1)
    # token by token
    dec = DecodeGraph(ctx, cfg, [bits(decode_layer(l, cfg)) for l in layers], cfg.batch, s_max=S)
    cache = decoder.new_cache(cfg, cfg.batch, S)
    xs = x0.reshape(cfg.batch, S, -1)
    eager = []
    for t in range(S):
        xt = np.ascontiguousarray(xs[:, t])
        _up(ctx, dec.x, oracle.to_bf16_bits(xt))
        dec.step()
        ctx.sync()
        eager.append(ctx.download(dec.out))
        got = oracle.from_bf16_bits(eager[-1])
        want = decoder.decode_step(cfg, xt, layers, cache, t, round_bf16=True)
        assert bf16_close(got, want) < 0, t
        assert bf16_close(got, prefill[:, t]) < 0, t
    assert int(ctx.download(dec.pos)[0]) == S                       # the device-side position advanced every step
    # the cache the steps built is the prefill's rotated K and V
    kc = oracle.from_bf16_bits(ctx.download(dec.kv[0]))
    assert bf16_close(kc[:cfg.batch], cache[0][0]) < 0 and bf16_close(kc[cfg.batch:], cache[0][1]) < 0
    # replay: the same step captured once into a CUDA graph gives the same bits, token after token
    rep = DecodeGraph(ctx, cfg, [bits(decode_layer(l, cfg)) for l in layers], cfg.batch, s_max=S)
    _up(ctx, rep.x, oracle.to_bf16_bits(np.ascontiguousarray(xs[:, 0])))
    rep.capture()                        # runs one eager step, then records the step
    rep.set_pos(0)
    launches = ctx.launches
    for t in range(S):
        _up(ctx, rep.x, oracle.to_bf16_bits(np.ascontiguousarray(xs[:, t])))
        rep.step()
        ctx.sync()
        assert np.array_equal(ctx.download(rep.out), eager[t]), t
    assert int(ctx.download(rep.pos)[0]) == S
    assert ctx.launches - launches >= 20 * S            # replayed kernels are counted as launches
    # a graph that has not run since it was planned cannot be captured
    from habu_b200.model_ir import HabuError
    fresh = DecodeGraph(ctx, cfg, [bits(decode_layer(l, cfg)) for l in layers], cfg.batch, s_max=S)
    with pytest.raises(HabuError):
        fresh.graph.capture()
    with pytest.raises(HabuError):
        fresh.graph.replay()
