"""Host-side logic of the tensor-parallel decoder without a GPU: shard arithmetic, and a
world-size-2 run over gloo in which each CPU rank evaluates its shard with the oracle
and the partial sums meet in an allreduce, compared with the unsharded oracle."""
import numpy as np
import pytest

from habu_b200.tp import DecoderConfig, check_shardable, shard_layer, shard_range
from mp_util import init_group, run_ranks

SMALL = DecoderConfig(d_model=128, n_q_heads=4, n_kv_heads=2, head_dim=32, ffn_hidden=256, n_layers=2, batch=2, seq=16)


def test_shard_ranges_cover_without_overlap():
    for world in (1, 2, 4, 8):
        spans = [shard_range(32, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 32
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    with pytest.raises(ValueError):
        shard_range(10, 4, 0)


def test_full_size_config_shards_up_to_eight_ranks():
    cfg = DecoderConfig()
    for world in (1, 2, 4, 8):
        check_shardable(cfg, world)
    assert cfg.n_q_heads // 8 == 4 and cfg.n_kv_heads // 8 == 1      # one KV head per rank, its 4 query heads local
    assert cfg.ffn_hidden // 8 == 1792
    with pytest.raises(ValueError):
        check_shardable(cfg, 16)
    assert abs(cfg.flops() - 7421.7e9) / 7421.7e9 < 1e-3


def test_shard_layer_keeps_gqa_groups_local_and_interleaves_gate_up():
    from oracle import decoder
    full = decoder.make_layer(SMALL, 0)
    hd = SMALL.head_dim
    parts = [shard_layer(full, SMALL, 2, r) for r in range(2)]
    for r, p in enumerate(parts):
        assert p["wqkv"].shape == ((2 + 2 * 1) * hd, 128) and p["wo"].shape == (128, 2 * hd)
        assert np.array_equal(p["wqkv"][:2 * hd], full["wq"][r * 2 * hd:(r + 1) * 2 * hd])
        assert np.array_equal(p["wqkv"][2 * hd:3 * hd], full["wk"][r * hd:(r + 1) * hd])
        assert np.array_equal(p["wqkv"][3 * hd:], full["wv"][r * hd:(r + 1) * hd])
        assert np.array_equal(p["wgu"][0::2], full["wg"][r * 128:(r + 1) * 128])
        assert np.array_equal(p["wgu"][1::2], full["wu"][r * 128:(r + 1) * 128])
        assert np.array_equal(p["wd"], full["wd"][:, r * 128:(r + 1) * 128])
    assert np.array_equal(np.concatenate([p["wo"] for p in parts], 1), full["wo"])


def _cpu_rank(rank, world):
    import torch
    import torch.distributed as dist
    from oracle import decoder
    init_group("gloo", rank, world)
    cfg = SMALL
    layers = [decoder.make_layer(cfg, i) for i in range(cfg.n_layers)]
    x0 = decoder.make_input(cfg)
    q0, q1 = shard_range(cfg.n_q_heads, world, rank)
    k0, k1 = shard_range(cfg.n_kv_heads, world, rank)
    f0, f1 = shard_range(cfg.ffn_hidden, world, rank)

    def reduce(a):
        t = torch.from_numpy(np.ascontiguousarray(a))
        dist.all_reduce(t)
        return t.numpy()
    got = decoder.forward(cfg, x0, layers, round_bf16=False, heads=(q0, q1, k0, k1), ffn=(f0, f1), reduce=reduce)
    ref = decoder.forward(cfg, x0, layers, round_bf16=False)
    assert np.allclose(got, ref, rtol=1e-4, atol=1e-4), float(np.abs(got - ref).max())
    # every rank ends with the same replicated residual stream
    gathered = [None] * world
    dist.all_gather_object(gathered, got.tobytes())
    assert all(g == gathered[0] for g in gathered)
    dist.destroy_process_group()


def test_two_cpu_ranks_over_gloo_match_the_unsharded_oracle():
    run_ranks(_cpu_rank, 2, timeout=240)


def test_candidate_schedules_are_well_formed():
    """The schedules the bench times: one rank needs none of the collective machinery; several
    ranks get the exposed schedule first (the safe fallback), the pipelined ones after it, and the
    gathered-product ones only on request."""
    from habu_b200.tp import candidate_schedules
    assert candidate_schedules(1) == [dict(chunks=1, fused=False)]
    for world in (2, 4, 8):
        c = candidate_schedules(world)
        assert c[0] == dict(chunks=1, fused=True, fused_form=1)
        assert all(s["fused"] and not s.get("gathered") for s in c)
        assert any(s["chunks"] == 2 and s["fused_form"] == 2 for s in c)
        g = candidate_schedules(world, gathered=True)
        assert g[:len(c)] == c and all(s["gathered"] and s["chunks"] == 1 and s["fused_form"] == 2 for s in g[len(c):])
        assert len(g) > len(c)
