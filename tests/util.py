"""Shared helpers for the parity tests: seeded bf16 inputs and error measures."""
import numpy as np

import oracle

SEED = 0x48414255  # "HABU"


def bf16_normal(shape, seed, std=1.0):
    """fp32 values already rounded to bf16, and their bit patterns."""
    x = oracle.round_bf16(oracle.normal(shape, seed, 0.0, std))
    return x, oracle.to_bf16_bits(x)


def max_abs(a, b):
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64))))


def max_rel(a, ref, eps=1e-3):
    """|a-ref| / max(|ref|, eps*max|ref|): relative error with a floor so that entries
    that cancel to ~0 are judged against the scale of the matrix."""
    ref = ref.astype(np.float64)
    floor = eps * float(np.max(np.abs(ref)))
    return float(np.max(np.abs(a.astype(np.float64) - ref) / np.maximum(np.abs(ref), floor)))
