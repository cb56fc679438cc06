"""CPU checks of the oracle itself.  The reference project has no implementation and no
golden vectors for this path (parity unpinned), so the oracle is checked against
independent numpy float64 evaluations and closed forms instead."""
import numpy as np

import oracle
from util import max_abs


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 1e-40, 0.0], np.float32)
    bits = oracle.to_bf16_bits(x)
    back = oracle.from_bf16_bits(bits)
    # 1 + 2^-8 is a tie between 1.0 and 1 + 2^-7 -> even (1.0); 1 + 3*2^-8 ties up to 1 + 2^-6
    assert back[0] == 1.0 and back[1] == 1.0 and back[2] == np.float32(1.015625)
    assert back[3] == -2.5
    y = x.copy()
    oracle.round_bf16(y)
    assert np.array_equal(y, back)


def test_generators_are_counter_based():
    a = oracle.normal((1000,), 7)
    b = oracle.normal((400,), 7, offset=600)
    assert np.array_equal(a[600:], b)
    u = oracle.uniform((100000,), 3)
    assert -1.0 <= u.min() and u.max() < 1.0 and abs(u.mean()) < 0.01
    n = oracle.normal((200000,), 5)
    assert abs(n.mean()) < 0.01 and abs(n.std() - 1.0) < 0.01


def test_gemm_matches_float64_all_layouts():
    A = oracle.normal((37, 70), 1)
    B = oracle.normal((70, 29), 2)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    for a in (A, np.ascontiguousarray(A.T).T):
        for b in (B, np.ascontiguousarray(B.T).T):
            assert max_abs(oracle.gemm(a, b), ref) < 2e-5
            assert max_abs(oracle.gemm(a, b, acc_double=True), ref) < 3e-6


def test_attention_matches_numpy_softmax():
    B, S, Hq, Hkv, D = 2, 33, 4, 2, 16
    Q, K, V = (oracle.normal(s, i) for i, s in enumerate([(B, S, Hq, D), (B, S, Hkv, D), (B, S, Hkv, D)]))
    for causal in (True, False):
        O, lse = oracle.attention(Q, K, V, causal=causal, return_lse=True)
        Kr, Vr = np.repeat(K, Hq // Hkv, 2).astype(np.float64), np.repeat(V, Hq // Hkv, 2).astype(np.float64)
        s = np.einsum("bihd,bjhd->bhij", Q.astype(np.float64), Kr) / np.sqrt(D)
        if causal:
            s = np.where(np.tril(np.ones((S, S), bool)), s, -np.inf)
        m = s.max(-1, keepdims=True)
        p = np.exp(s - m)
        ref = np.einsum("bhij,bjhd->bihd", p / p.sum(-1, keepdims=True), Vr)
        assert max_abs(O, ref) < 2e-6
        assert max_abs(lse, (m + np.log(p.sum(-1, keepdims=True)))[..., 0]) < 1e-5
        assert abs((p / p.sum(-1, keepdims=True)).sum(-1) - 1).max() < 1e-12


def test_rope_preserves_norm_and_is_identity_at_position_zero():
    x = oracle.normal((12, 4 * 32), 9)
    y = oracle.rope(x, seq=6, heads=4, head_dim=32)
    assert np.allclose(np.linalg.norm(x.reshape(12, 4, 32), axis=-1), np.linalg.norm(y.reshape(12, 4, 32), axis=-1), rtol=1e-5)
    assert np.array_equal(y[0], x[0]) and np.array_equal(y[6], x[6])
    # closed form for one pair
    t, h, i, d = 5, 2, 3, 32
    th = 5 * 10000.0 ** (-2 * i / d)
    a, b = x[t, h * d + i], x[t, h * d + i + d // 2]
    assert abs(y[t, h * d + i] - (a * np.cos(th) - b * np.sin(th))) < 1e-6


def test_rmsnorm_swiglu_gelu_argmax_embedding():
    x = oracle.normal((5, 64), 11)
    g = oracle.uniform((64,), 12, 0.5, 1.5)
    ref = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-5) * g
    assert max_abs(oracle.rmsnorm(x, g), ref) < 1e-6
    sw = oracle.swiglu(x)
    assert max_abs(sw, x[:, :32] / (1 + np.exp(-x[:, :32].astype(np.float64))) * x[:, 32:]) < 1e-6
    inter = np.empty_like(x)
    inter[:, 0::2], inter[:, 1::2] = x[:, :32], x[:, 32:]
    assert np.array_equal(oracle.swiglu(inter, interleaved=True), sw)
    from math import erf
    assert max_abs(oracle.gelu(x), np.vectorize(lambda v: 0.5 * v * (1 + erf(v / np.sqrt(2))))(x.astype(np.float64))) < 1e-6
    h = 1e-3
    num = (oracle.gelu(x + h).astype(np.float64) - oracle.gelu(x - h)) / (2 * h)
    assert max_abs(oracle.gelu_backward(x, np.ones_like(x)), num) < 1e-3
    assert np.array_equal(oracle.argmax(x), x.argmax(-1).astype(np.int32))
    tie = np.zeros((1, 8), np.float32)
    assert oracle.argmax(tie)[0] == 0
    ids = np.array([3, 0, 3, 4], np.int32)
    assert np.array_equal(oracle.embedding(x, ids), x[ids])


def test_adam_first_step_closed_form_and_mse():
    w = oracle.normal((1000,), 21)
    g = oracle.normal((1000,), 22)
    w0 = w.copy()
    m = np.zeros_like(w)
    v = np.zeros_like(w)
    oracle.adam(w, m, v, g, lr=1e-3, step=1)
    # after bias correction the first step is lr * g / (|g| + eps)
    assert max_abs(w, w0 - 1e-3 * g / (np.abs(g) + 1e-8)) < 1e-6
    assert abs(oracle.mse(w, w0) - float(((w.astype(np.float64) - w0) ** 2).mean())) < 1e-12


def test_all_reduce_sums_in_rank_order():
    bufs = [oracle.normal((257,), 30 + r) for r in range(4)]
    ref = bufs[0].copy()
    for b in bufs[1:]:
        ref = ref + b
    oracle.all_reduce(bufs)
    for b in bufs:
        assert np.array_equal(b, ref)
