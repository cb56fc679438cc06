"""CPU restatement of the MLP training step (test infrastructure only; parity unpinned:
the reference project has no such path).  n layers y = x @ W^T without biases, erf-GELU
between layers and none after the last, MSE = mean over all elements, bias-corrected Adam
without weight decay.  Tensors the device stores in bf16 are rounded at the same points
when round_bf16 is set."""
from __future__ import annotations

import numpy as np

import oracle

SEED = 0x48414255


def make_weights(width, n_layers, seed=SEED):
    """fp32 master weights [out, in] ~ N(0, 1/width) (variance-preserving init)."""
    return [oracle.normal((width, width), seed + 500 + i, 0.0, width ** -0.5) for i in range(n_layers)]


def make_batch(batch, width, rank=0, seed=SEED):
    x = oracle.round_bf16(oracle.normal((batch, width), seed + 600 + 10 * rank))
    y = oracle.round_bf16(oracle.normal((batch, width), seed + 601 + 10 * rank))
    return x, y


def forward_backward(ws_bf16, x, y, round_bf16=True):
    """Returns (loss, grads) with grads[i] = dL/dW_i ([out, in])."""
    rnd = (lambda a: oracle.round_bf16(np.ascontiguousarray(a, np.float32))) if round_bf16 else (lambda a: np.ascontiguousarray(a, np.float32))
    n = len(ws_bf16)
    hs, zs = [x], []
    for i, w in enumerate(ws_bf16):
        z = rnd(oracle.gemm(hs[-1], w.T))
        zs.append(z)
        if i < n - 1:
            hs.append(rnd(oracle.gelu(z)))
    loss = oracle.mse(zs[-1], y)
    d = rnd((zs[-1] - y) * np.float32(2.0 / y.size))
    grads = [None] * n
    for i in reversed(range(n)):
        grads[i] = rnd(oracle.gemm(np.ascontiguousarray(d.T), hs[i]))
        if i > 0:
            dh = rnd(oracle.gemm(d, ws_bf16[i]))
            d = rnd(oracle.gelu_backward(zs[i - 1], dh))
    return loss, grads


def adam_update(w32, m, v, grads, step, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, grad_scale=1.0):
    for w, mm, vv, g in zip(w32, m, v, grads):
        oracle.adam(w.reshape(-1), mm.reshape(-1), vv.reshape(-1), np.ascontiguousarray(g * np.float32(grad_scale)).reshape(-1),
                    lr, b1, b2, eps, step)
