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
