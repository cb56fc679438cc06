"""Writes tests/golden/oracle_small.npz: outputs of the CPU oracle on small seeded cases.

The reference project has no implementation of this path, so these are NOT reference
outputs; they pin the oracle itself (and the seeded generators) against accidental change,
and give the GPU tests a fixed set of expected values that does not depend on rebuilding
the oracle.  Inputs are not stored: each case regenerates them from its seed with the
counter-based generators, exactly as the tests do.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import oracle  # noqa: E402
from util import SEED, bf16_normal  # noqa: E402


def cases():
    """name -> (inputs dict, expected output).  Shared with tests/test_y_golden.py."""
    out = {}
    # bf16 GEMM 128 x 256 x 64, B column-major (given as [N, K])
    A, _ = bf16_normal((128, 64), SEED + 1, 64 ** -0.5)
    Bt, _ = bf16_normal((256, 64), SEED + 2, 1.0)
    out["gemm_bf16_128x256x64"] = ({"A": A, "Bt": Bt}, oracle.gemm(A, Bt.T))
    # fp32 GEMM 100 x 37 x 50 with double accumulation
    A32 = oracle.uniform((100, 50), SEED + 21)
    B32 = oracle.uniform((50, 37), SEED + 22)
    out["gemm_f32_100x37x50"] = ({"A": A32, "B": B32}, oracle.gemm(A32, B32, acc_double=True))
    # causal grouped-query attention, ragged sequence
    Q, _ = bf16_normal((1, 136, 2, 128), SEED + 31)
    K, _ = bf16_normal((1, 136, 1, 128), SEED + 32)
    V, _ = bf16_normal((1, 136, 1, 128), SEED + 33)
    out["attention_causal_gqa_s136"] = ({"Q": Q, "K": K, "V": V}, oracle.attention(Q, K, V, causal=True))
    # glue
    x, _ = bf16_normal((24, 256), SEED + 41)
    g = oracle.round_bf16(oracle.uniform((256,), SEED + 42, 0.5, 1.5))      # the device keeps gains in bf16
    out["rmsnorm_24x256"] = ({"x": x, "g": g}, oracle.rmsnorm(x, g, 1e-5))
    r, _ = bf16_normal((2 * 12, 2 * 128), SEED + 43)
    out["rope_s12_h2_d128"] = ({"x": r}, oracle.rope(r, 12, 2, 128, 10000.0))
    gu, _ = bf16_normal((32, 512), SEED + 44)
    out["swiglu_32x512"] = ({"x": gu}, oracle.swiglu(gu))
    out["gelu_24x256"] = ({"x": x}, oracle.gelu(x))
    return out


if __name__ == "__main__":
    arrays = {name: exp.astype(np.float32) for name, (_, exp) in cases().items()}
    path = os.path.join(HERE, "oracle_small.npz")
    np.savez_compressed(path, **arrays)
    print(path, {k: v.shape for k, v in arrays.items()}, os.path.getsize(path), "bytes")
