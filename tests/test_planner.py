"""Memory planner placement rule (`hb_plan_arena`), checked on the CPU: property tests over
random lifetimes plus the decoder block's own tensor list."""
import numpy as np
import pytest

from habu_b200.graph import plan_arena

ALIGN = 256
up = lambda x: (x + ALIGN - 1) // ALIGN * ALIGN


def check(sizes, first, last, offs, total):
    n = len(sizes)
    assert all(o % ALIGN == 0 for o in offs)
    for i in range(n):
        assert offs[i] + up(sizes[i]) <= total
        for j in range(i):
            alive_together = not (last[i] < first[j] or last[j] < first[i])
            overlap = offs[i] < offs[j] + up(sizes[j]) and offs[j] < offs[i] + up(sizes[i])
            assert not (alive_together and overlap), (i, j)
    # bounds: at least the heaviest instant, at most everything side by side
    steps = max(last) + 1 if n else 0
    peak = max((sum(up(sizes[i]) for i in range(n) if first[i] <= s <= last[i]) for s in range(steps)), default=0)
    assert peak <= total <= sum(up(s) for s in sizes)
    return peak


@pytest.mark.parametrize("seed", range(8))
def test_random_lifetimes_never_alias_and_stay_within_bounds(seed):
    rng = np.random.default_rng(seed)
    n = int(rng.integers(1, 60))
    steps = int(rng.integers(1, 40))
    sizes = [int(x) for x in rng.integers(1, 1 << 20, n)]
    first = [int(x) for x in rng.integers(0, steps, n)]
    last = [min(steps - 1, f + int(d)) for f, d in zip(first, rng.integers(0, 6, n))]
    offs, total = plan_arena(sizes, first, last)
    check(sizes, first, last, offs, total)
    assert plan_arena(sizes, first, last) == (offs, total)        # deterministic


def test_chain_of_temporaries_reuses_two_slots():
    # x0 -> x1 -> x2 -> ...: each temporary dies as soon as the next node has read it
    n = 12
    sizes = [1 << 20] * n
    first = list(range(n))
    last = [i + 1 for i in range(n)]
    offs, total = plan_arena(sizes, first, last)
    check(sizes, first, last, offs, total)
    assert total == 2 << 20
    assert sorted(set(offs)) == [0, 1 << 20]


def test_decoder_block_activations_fit_the_peak_not_the_sum():
    # one Llama-style block at 8192 tokens, d_model 4096, hidden 14336 (bytes of bf16 tensors);
    # node order: norm, qkv, rope, attention, wo, add, norm, gate/up (SwiGLU fused), down, add
    T, d, f, kv = 8192, 4096, 14336, 1024
    t = lambda cols: T * cols * 2
    sizes = [t(d), t(d + 2 * kv), t(d), t(d), t(d), t(d), t(f), t(d), t(d)]
    first = [0, 1, 3, 4, 5, 6, 7, 8, 9]
    last = [1, 3, 4, 5, 6, 7, 8, 9, 9]
    offs, total = plan_arena(sizes, first, last)
    peak = check(sizes, first, last, offs, total)
    assert total < 0.5 * sum(sizes)
    assert total <= 1.25 * peak


def test_degenerate_inputs():
    assert plan_arena([], [], []) == ([], 0)
    offs, total = plan_arena([1], [0], [0])
    assert (offs, total) == ([0], 256)
    with pytest.raises(ValueError):
        plan_arena([16], [3], [2])          # dies before it is born
    with pytest.raises(ValueError):
        plan_arena([16], [-1], [2])


# ---- default routing of bf16 matmuls (host arithmetic of the dispatcher)
def test_default_route_of_the_configured_shapes():
    from habu_b200.model_ir import matmul_default_route, matmul_configs
    cfgs = matmul_configs()
    for s in (4096, 8192):                       # a 256 x 256 tile for every pair of SMs: CTA-pair kernel
        r = matmul_default_route(s, s, s)
        assert r.kernel == 1 and cfgs[r.config_id].cluster == 2 and cfgs[r.config_id].tile_m == 256
    r = matmul_default_route(1024, 1024, 1024)   # 16 pair tiles for 74 pairs: one-CTA tiles instead
    assert r.kernel == 0 and cfgs[r.config_id].cluster == 1
    assert (1024 // 128) * (1024 // cfgs[r.config_id].tile_n) >= 64
    # M-major or N-major operands and fused epilogues never take the stream-K path
    assert matmul_default_route(16, 8192, 8192, layout=2).kernel != 2
    assert matmul_default_route(16, 8192, 8192, epilogue=1).kernel != 2


@pytest.mark.parametrize("m,n,k", [(16, 8192, 8192), (1, 256, 512), (7, 1000, 1096), (33, 4096, 2048), (64, 384, 8192),
                                   (64, 128 * 1024, 64)])
def test_stream_k_plan_covers_the_work_within_its_scratch(m, n, k):
    from habu_b200.model_ir import matmul_default_route
    r = matmul_default_route(m, n, k)
    assert r.kernel == 2 and r.config_id == -1
    tiles = -(-n // 128)
    assert r.tiles == tiles
    assert 1 <= r.grid <= 148
    assert 2 <= r.max_segments <= max(2, r.grid)
    mpad = -(-m // 16) * 16
    assert r.scratch_bytes == tiles * r.max_segments * 128 * mpad * 4
    # a K range never spans more tiles than the segments reserved for one tile allow:
    # with `units` (tile, k-group) pairs dealt out evenly, a CTA's range is at least units // grid long
    k_groups = -(-k // 128)
    units = tiles * k_groups
    shortest = units // r.grid
    assert shortest >= 1
    assert -(-k_groups // shortest) + 1 <= r.max_segments or r.max_segments == r.grid


def test_output_staging_swizzle_is_the_64_byte_tma_pattern():
    """The GEMM epilogue writes piece c (16 bytes) of row r of a 32 x 32 bf16 block at
    r*64 + ((c ^ ((r >> 1) & 3)) << 4) and stores the block with a 64-byte-swizzled tensor map.
    That must be the hardware's pattern (address bits 4-5 xor-ed with bits 7-8 of a 512-byte
    aligned buffer), fill the 2 KB buffer exactly once, and let the eight lanes of a quarter
    warp hit eight different 16-byte bank groups."""
    seen = set()
    for r in range(32):
        for c in range(4):
            off = r * 64 + ((c ^ ((r >> 1) & 3)) << 4)
            linear = r * 64 + c * 16                      # where the piece sits in the unswizzled block
            assert off == linear ^ (((linear >> 7) & 3) << 4)
            seen.add(off)
    assert seen == set(range(0, 2048, 16))
    for c in range(4):
        for r0 in range(0, 32, 8):
            groups = {((r * 64 + ((c ^ ((r >> 1) & 3)) << 4)) % 128) // 16 for r in range(r0, r0 + 8)}
            assert len(groups) == 8
