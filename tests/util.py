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


def bf16_close(got, ref, atol=2e-2, rel=2.0 ** -8):
    """Largest excess over the bf16-path tolerance: max-abs `atol` against the fp32
    reference, widened by one bf16 output rounding (`rel` = 2^-8 relative) where |ref| is large."""
    ref = ref.astype(np.float64)
    return float(np.max(np.abs(got.astype(np.float64) - ref) - (atol + np.abs(ref) * rel)))


def max_rel(a, ref, eps=1e-3):
    """|a-ref| / max(|ref|, eps*max|ref|): relative error with a floor so that entries
    that cancel to ~0 are measured against the scale of the matrix."""
    ref = ref.astype(np.float64)
    floor = eps * float(np.max(np.abs(ref)))
    return float(np.max(np.abs(a.astype(np.float64) - ref) / np.maximum(np.abs(ref), floor)))
