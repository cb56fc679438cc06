"""Runs the autotune entry point over a list of matmul shapes and persists the winners.

    python -m habu_b200.tune                 # the benchmark configurations' shapes
    python -m habu_b200.tune 4096x4096x4096  # M x N x K [x layout [x epilogue]]

The cache (``habu_b200/tune_cache.txt``, one text line per operator, shape, SM count and GPU
name, the choice written by its properties) is loaded by every :class:`habu_b200.Context` at
creation; shapes without an entry use the heuristic in the library.
"""
from __future__ import annotations

import os
import sys

CACHE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tune_cache.txt")

# (M, N, K, layout, epilogue): bench GEMMs, the decoder's projections at TP 1/2/4/8 (also per
# row block of 4096 and 2048 tokens) and the MLP's forward / dW / dX products.
def default_shapes():
    shapes = [(1024, 1024, 1024, 0, 0), (4096, 4096, 4096, 0, 0), (8192, 8192, 8192, 0, 0)]
    for tp in (1, 2, 4, 8):
        for T in (8192, 4096, 2048):
            shapes += [(T, 6144 // tp, 4096, 0, 0), (T, 4096, 4096 // tp, 0, 0),
                       (T, 2 * 14336 // tp, 4096, 0, 2), (T, 4096, 14336 // tp, 0, 0)]
    shapes += [(4096, 8192, 8192, 0, 0), (8192, 8192, 4096, 3, 0), (4096, 8192, 8192, 2, 0)]
    seen, out = set(), []
    for s in shapes:
        if s not in seen:
            seen.add(s)
            out.append(s)
    return out


# Decode-shaped products (M = 16 new tokens) of the same block, and the attention shapes of the
# benchmark and of the decoder at TP 1/2/4/8: (batch, seq, q heads, kv heads, causal).
def default_skinny_shapes():
    return [(16, 8192, 8192), (16, 6144, 4096), (16, 4096, 4096), (16, 28672, 4096), (16, 4096, 14336)]


def default_attention_shapes():
    return [(8, 4096, 32, 8, True)] + [(4, 2048, 32 // tp, 8 // tp, True) for tp in (1, 2, 4, 8)]


def main(argv):
    import habu_b200 as hb
    ctx = hb.Context(0, load_tune_cache=False)
    if os.path.exists(CACHE):
        ctx.tune_cache_load(CACHE)
    shapes = [tuple(int(x) for x in a.split("x")) + (0, 0) for a in argv] or default_shapes()
    for s in shapes:
        m, n, k, layout, epi = s[:5]
        r = ctx.autotune(m, n, k, layout, epi, search=True)
        print(f"{m}x{n}x{k} layout {layout} epilogue {epi}: config {r.config_id} (cluster {r.cluster}, tile "
              f"{r.tile_m}x{r.tile_n}x{r.tile_k}, {r.stages} stages, raster {r.raster_group}) {r.ms * 1e3:.1f} us "
              f"{r.tflops:.0f} TFLOP/s", flush=True)
    if not argv:
        for m, n, k in default_skinny_shapes():
            r = ctx.autotune(m, n, k, search=True)
            print(f"{m}x{n}x{k} stream-K: grid {r.split_k}, {r.tile_k // 64} k-blocks per stage, {r.ms * 1e3:.1f} us "
                  f"{2.0 * (m * k + n * k + m * n) / (r.ms * 1e-3) / 1e9:.0f} GB/s", flush=True)
        for b, s_, hq, hkv, causal in default_attention_shapes():
            r = ctx.autotune_attention(b, s_, hq, hkv, causal, search=True)
            print(f"attention batch {b} seq {s_} heads {hq}/{hkv}: {'persistent' if r.config_id else 'one unit per CTA'} "
                  f"{r.ms * 1e3:.1f} us {r.tflops:.0f} TFLOP/s", flush=True)
    ctx.tune_cache_save(CACHE)
    print(f"saved {CACHE}")


if __name__ == "__main__":
    main(sys.argv[1:])
