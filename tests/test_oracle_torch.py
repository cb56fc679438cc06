"""Independent cross-check of the CPU oracle against PyTorch on the CPU.

The oracle has no reference implementation to be pinned on (the reference project has no
tensor code), so its definitions are checked here against a second, independently written
implementation: torch's own matmul, scaled_dot_product_attention, rms norm written from the
formula, erf-GELU, SiLU, Adam optimiser and autograd.  float64 torch is the yardstick for
the fp32 oracle (tolerance 1e-4 relative unless stated).
"""
import types

import numpy as np
import pytest
import torch

import oracle
from oracle import decoder as odec
from oracle import mlp as omlp
from util import SEED, max_abs, max_rel

t64 = lambda a: torch.from_numpy(np.asarray(a, np.float64))


def test_gemm_and_attention_match_torch():
    A = oracle.normal((96, 72), SEED + 1)
    B = oracle.normal((72, 40), SEED + 2)
    assert max_rel(oracle.gemm(A, B), (t64(A) @ t64(B)).numpy()) < 1e-4
    Bt, S, Hq, Hkv, D = 2, 77, 4, 2, 32
    Q = oracle.normal((Bt, S, Hq, D), SEED + 3)
    K = oracle.normal((Bt, S, Hkv, D), SEED + 4)
    V = oracle.normal((Bt, S, Hkv, D), SEED + 5)
    for causal in (True, False):
        got, lse = oracle.attention(Q, K, V, causal=causal, return_lse=True)
        q, k, v = (t64(x).permute(0, 2, 1, 3) for x in (Q, K, V))      # [B, H, S, D]
        k = k.repeat_interleave(Hq // Hkv, dim=1)                      # grouped-query heads
        v = v.repeat_interleave(Hq // Hkv, dim=1)
        ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal)
        assert max_abs(got, ref.permute(0, 2, 1, 3).numpy()) < 1e-5
        s = (q @ k.transpose(-1, -2)) * D ** -0.5
        if causal:
            s = s.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
        assert max_abs(lse, torch.logsumexp(s, -1).numpy()) < 1e-4


def _rotate_half_rope(x, seq, heads, hd, base):
    """Textbook rotate-half RoPE in torch: pairs (i, i + hd/2), theta_i = base^(-2i/hd)."""
    tokens = x.shape[0]
    x = x.reshape(tokens, heads, hd)
    pos = (torch.arange(tokens) % seq).double()
    inv = base ** (-torch.arange(0, hd, 2).double() / hd)
    ang = pos[:, None] * inv[None, :]                                   # [tokens, hd/2]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., : hd // 2], x[..., hd // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], -1).reshape(tokens, heads * hd)


def test_glue_ops_match_torch():
    x = oracle.normal((24, 64), SEED + 6)
    g = oracle.uniform((64,), SEED + 7, 0.5, 1.5)
    X = t64(x)
    ref = X * torch.rsqrt((X * X).mean(-1, keepdim=True) + 1e-5) * t64(g)
    assert max_rel(oracle.rmsnorm(x, g, 1e-5), ref.numpy()) < 1e-4
    assert max_abs(oracle.gelu(x), torch.nn.functional.gelu(X).numpy()) < 1e-5     # erf form
    gu = oracle.normal((24, 128), SEED + 8)
    G, U = t64(gu[:, :64]), t64(gu[:, 64:])
    assert max_abs(oracle.swiglu(gu), (torch.nn.functional.silu(G) * U).numpy()) < 1e-5
    inter = np.empty_like(gu)
    inter[:, 0::2], inter[:, 1::2] = gu[:, :64], gu[:, 64:]
    assert max_abs(oracle.swiglu(inter, interleaved=True), (torch.nn.functional.silu(G) * U).numpy()) < 1e-5
    r = oracle.normal((2 * 12, 4 * 16), SEED + 9)
    assert max_abs(oracle.rope(r, 12, 4, 16, 10000.0), _rotate_half_rope(t64(r), 12, 4, 16, 10000.0).numpy()) < 1e-4
    # GELU derivative against autograd
    Xg = X.clone().requires_grad_(True)
    dy = oracle.normal(x.shape, SEED + 10)
    torch.nn.functional.gelu(Xg).backward(t64(dy))
    assert max_abs(oracle.gelu_backward(x, dy), Xg.grad.numpy()) < 1e-5
    y, t = oracle.normal((8, 32), SEED + 11), oracle.normal((8, 32), SEED + 12)
    assert abs(oracle.mse(y, t) - float(torch.nn.functional.mse_loss(t64(y), t64(t)))) < 1e-6


def test_adam_matches_torch_optimizer_over_several_steps():
    n = 257
    w = oracle.normal((n,), SEED + 13)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    p = torch.nn.Parameter(t64(w).clone())
    opt = torch.optim.Adam([p], lr=1e-3, betas=(0.9, 0.999), eps=1e-8)
    for step in range(1, 6):
        g = oracle.normal((n,), SEED + 20 + step)
        oracle.adam(w, m, v, g, 1e-3, 0.9, 0.999, 1e-8, step)
        p.grad = t64(g).clone()
        opt.step()
        assert max_abs(w, p.detach().numpy()) < 1e-6, step


def test_mlp_forward_backward_matches_autograd():
    width, batch, layers = 48, 16, 3
    ws = [oracle.round_bf16(w) for w in omlp.make_weights(width, layers)]
    x, y = omlp.make_batch(batch, width)
    loss, grads = omlp.forward_backward(ws, x, y, round_bf16=False)
    Ws = [t64(w).requires_grad_(True) for w in ws]
    h = t64(x)
    for i, W in enumerate(Ws):
        h = h @ W.T
        if i < layers - 1:
            h = torch.nn.functional.gelu(h)
    L = torch.nn.functional.mse_loss(h, t64(y))
    L.backward()
    assert abs(loss - L.item()) < 1e-5 * max(1.0, abs(L.item()))
    for g, W in zip(grads, Ws):
        assert max_rel(g, W.grad.numpy()) < 1e-3


def test_decoder_block_matches_torch_model():
    cfg = types.SimpleNamespace(d_model=64, n_q_heads=4, n_kv_heads=2, head_dim=16, ffn_hidden=96, batch=2, seq=10,
                                eps=1e-5, rope_base=10000.0, tokens=20)
    layers = [odec.make_layer(cfg, i) for i in range(2)]
    # unit gains hide the gain path: perturb them
    for i, lw in enumerate(layers):
        lw["g1"] = oracle.uniform((cfg.d_model,), SEED + 30 + i, 0.5, 1.5)
        lw["g2"] = oracle.uniform((cfg.d_model,), SEED + 40 + i, 0.5, 1.5)
    x0 = odec.make_input(cfg)
    got = odec.forward(cfg, x0, layers, round_bf16=False)
    B, S, hd = cfg.batch, cfg.seq, cfg.head_dim
    norm = lambda X, g: X * torch.rsqrt((X * X).mean(-1, keepdim=True) + cfg.eps) * t64(g)
    x = t64(x0)
    for lw in layers:
        h = norm(x, lw["g1"])
        q = _rotate_half_rope(h @ t64(lw["wq"]).T, S, cfg.n_q_heads, hd, cfg.rope_base)
        k = _rotate_half_rope(h @ t64(lw["wk"]).T, S, cfg.n_kv_heads, hd, cfg.rope_base)
        v = h @ t64(lw["wv"]).T
        sh = lambda X, H: X.reshape(B, S, H, hd).permute(0, 2, 1, 3)
        rep = cfg.n_q_heads // cfg.n_kv_heads
        a = torch.nn.functional.scaled_dot_product_attention(
            sh(q, cfg.n_q_heads), sh(k, cfg.n_kv_heads).repeat_interleave(rep, 1),
            sh(v, cfg.n_kv_heads).repeat_interleave(rep, 1), is_causal=True)
        a = a.permute(0, 2, 1, 3).reshape(B * S, cfg.n_q_heads * hd)
        x = x + a @ t64(lw["wo"]).T
        h2 = norm(x, lw["g2"])
        x = x + (torch.nn.functional.silu(h2 @ t64(lw["wg"]).T) * (h2 @ t64(lw["wu"]).T)) @ t64(lw["wd"]).T
    got = got[0] if isinstance(got, tuple) else got
    assert max_abs(got, x.numpy()) < 1e-4
