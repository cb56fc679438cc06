"""CPU restatement of the Llama-style decoder block forward (test infrastructure only).

No reference implementation exists (parity unpinned); this follows the configuration's
definition: pre-norm blocks, RMSNorm eps 1e-5 with gain, rotate-half RoPE base 10000,
grouped-query causal attention with scale 1/sqrt(head_dim), SwiGLU FFN, residual adds.
``round_bf16=True`` rounds every tensor the device stores in bf16 at the same points
(the "bf16-storage" mode); ``False`` keeps fp32 throughout (the fp32 reference).
"""
from __future__ import annotations

import numpy as np

import oracle

SEED = 0x48414255


def make_layer(cfg, layer: int, seed: int = SEED):
    """Full (unsharded) weights of one layer, N(0, 0.02) rounded to bf16, gains = 1.
    Each matrix is [out_features, in_features]."""
    d, hd = cfg.d_model, cfg.head_dim
    s = seed + 100 * (layer + 1)
    mk = lambda shape, k: oracle.round_bf16(oracle.normal(shape, s + k, 0.0, 0.02))
    return {"wq": mk((cfg.n_q_heads * hd, d), 1), "wk": mk((cfg.n_kv_heads * hd, d), 2),
            "wv": mk((cfg.n_kv_heads * hd, d), 3), "wo": mk((d, cfg.n_q_heads * hd), 4),
            "wg": mk((cfg.ffn_hidden, d), 5), "wu": mk((cfg.ffn_hidden, d), 6), "wd": mk((d, cfg.ffn_hidden), 7),
            "g1": np.ones(d, np.float32), "g2": np.ones(d, np.float32)}


def make_input(cfg, seed: int = SEED):
    return oracle.round_bf16(oracle.normal((cfg.tokens, cfg.d_model), seed + 7))


def forward(cfg, x0, layers, round_bf16=True, heads=None, ffn=None, reduce=None, residual_fp32=False):
    """Decoder forward.  `heads=(q0,q1,k0,k1)` and `ffn=(f0,f1)` restrict the computation
    to one rank's shard, in which case `reduce` (a function summing partials across
    ranks) must be given; with all three None the whole model is evaluated.
    `residual_fp32` (bf16-storage mode only): the residual stream x is kept in fp32, as the
    device keeps it; sublayer outputs are still rounded to bf16 before they are added."""
    rnd = (lambda a: oracle.round_bf16(np.ascontiguousarray(a, np.float32))) if round_bf16 else (lambda a: np.ascontiguousarray(a, np.float32))
    hd, B, S = cfg.head_dim, cfg.batch, cfg.seq
    q0, q1, k0, k1 = heads if heads else (0, cfg.n_q_heads, 0, cfg.n_kv_heads)
    f0, f1 = ffn if ffn else (0, cfg.ffn_hidden)
    reduce = reduce or (lambda a: a)
    rnd_x = (lambda a: np.ascontiguousarray(a, np.float32)) if residual_fp32 else rnd
    x = x0.astype(np.float32)
    for lw in layers:
        h = rnd(oracle.rmsnorm(x, lw["g1"], cfg.eps))
        q = rnd(oracle.gemm(h, lw["wq"][q0 * hd:q1 * hd].T))
        k = rnd(oracle.gemm(h, lw["wk"][k0 * hd:k1 * hd].T))
        v = rnd(oracle.gemm(h, lw["wv"][k0 * hd:k1 * hd].T))
        q = rnd(oracle.rope(q, S, q1 - q0, hd, cfg.rope_base))
        k = rnd(oracle.rope(k, S, k1 - k0, hd, cfg.rope_base))
        a = oracle.attention(q.reshape(B, S, q1 - q0, hd), k.reshape(B, S, k1 - k0, hd), v.reshape(B, S, k1 - k0, hd),
                             causal=True, round_p=round_bf16)
        a = rnd(a.reshape(B * S, (q1 - q0) * hd))
        ao = reduce(rnd(oracle.gemm(a, np.ascontiguousarray(lw["wo"][:, q0 * hd:q1 * hd]).T)))
        x = rnd_x(x + rnd(ao))
        h2 = rnd(oracle.rmsnorm(x, lw["g2"], cfg.eps))
        g = oracle.gemm(h2, lw["wg"][f0:f1].T)
        u = oracle.gemm(h2, lw["wu"][f0:f1].T)
        act = rnd(oracle.swiglu(np.concatenate([g, u], 1)))
        fo = reduce(rnd(oracle.gemm(act, np.ascontiguousarray(lw["wd"][:, f0:f1]).T)))
        x = rnd_x(x + rnd(fo))
    return x


def new_cache(cfg, batch, s_max):
    """Per layer: (K, V), each [batch, s_max, n_kv_heads, head_dim] fp32, zero-filled."""
    return [(np.zeros((batch, s_max, cfg.n_kv_heads, cfg.head_dim), np.float32),
             np.zeros((batch, s_max, cfg.n_kv_heads, cfg.head_dim), np.float32)) for _ in range(cfg.n_layers)]


def decode_step(cfg, x_t, layers, cache, pos, round_bf16=True):
    """One generation step: x_t [batch, d_model] are the new tokens' embeddings at position
    `pos` of every sequence; `cache` (from :func:`new_cache`) holds the rotated keys and the
    values of positions < pos and receives those of `pos`.  Same definitions as :func:`forward`
    (the step for token t reproduces row t of the prefill forward of the same sequence); in
    bf16-storage mode the roundings sit where the device's decode graph stores bf16: gate and up
    projections are rounded before SwiGLU (a stand-alone kernel there), the residual stream after
    every add."""
    rnd = (lambda a: oracle.round_bf16(np.ascontiguousarray(a, np.float32))) if round_bf16 else (lambda a: np.ascontiguousarray(a, np.float32))
    hd, Hq, Hkv = cfg.head_dim, cfg.n_q_heads, cfg.n_kv_heads
    B = x_t.shape[0]
    G = Hq // Hkv
    x = x_t.astype(np.float32)
    scale = np.float32(1.0 / np.sqrt(hd))
    for lw, (Kc, Vc) in zip(layers, cache):
        h = rnd(oracle.rmsnorm(x, lw["g1"], cfg.eps))
        q = rnd(oracle.gemm(h, lw["wq"].T))
        k = rnd(oracle.gemm(h, lw["wk"].T))
        v = rnd(oracle.gemm(h, lw["wv"].T))
        q = rnd(oracle.rope(q, 1, Hq, hd, cfg.rope_base, pos0=pos))       # one token per row, all at position pos
        k = rnd(oracle.rope(k, 1, Hkv, hd, cfg.rope_base, pos0=pos))
        Kc[:, pos] = k.reshape(B, Hkv, hd)
        Vc[:, pos] = v.reshape(B, Hkv, hd)
        L = pos + 1
        qh = q.reshape(B, Hkv, G, hd)
        s = np.einsum("bkgd,blkd->bkgl", qh, Kc[:, :L], dtype=np.float32) * scale
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s, dtype=np.float32)
        p = p / p.sum(-1, keepdims=True)
        a = rnd(np.einsum("bkgl,blkd->bkgd", p, Vc[:, :L], dtype=np.float32).reshape(B, Hq * hd))
        ao = rnd(oracle.gemm(a, lw["wo"].T))
        x = rnd(x + ao)
        h2 = rnd(oracle.rmsnorm(x, lw["g2"], cfg.eps))
        gu = np.concatenate([rnd(oracle.gemm(h2, lw["wg"].T)), rnd(oracle.gemm(h2, lw["wu"].T))], 1)
        act = rnd(oracle.swiglu(gu))
        fo = rnd(oracle.gemm(act, lw["wd"].T))
        x = rnd(x + fo)
    return x
