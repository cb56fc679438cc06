"""Autotune cache: the persisted text format round-trips (no GPU needed for the file
checks), and on a GPU a search records a winner that the cached mode then returns."""
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CACHE = os.path.join(ROOT, "habu_b200", "tune_cache.txt")


def test_committed_cache_is_well_formed():
    """Version-2 lines name a choice by its properties; every matmul line must resolve to a
    configuration this build has (so the committed cache is never silently ignored)."""
    text = open(CACHE).read()
    assert text.startswith("# habu_b200 autotune cache v2")
    lines = [l for l in text.splitlines() if l and not l.startswith("#")]
    assert len(lines) >= 10
    import habu_b200
    have = {(c.cluster, c.tile_m, c.tile_n, c.tile_k, c.stages, c.raster_group) for c in habu_b200.matmul_configs()}
    for l in lines:
        key, val = l.split(" = ")
        op, dtype, m, n, k, layout, epi, sm, gpu = key.split()
        assert op in ("matmul", "skinny", "attention") and dtype == "bf16" and sm.startswith("sm") and " " not in gpu
        assert all(int(x) > 0 for x in (m, n, k))
        f = val.split()
        assert float(f[f.index("ms") + 1]) > 0
        if op == "matmul":
            assert 0 <= int(layout) <= 3 and 0 <= int(epi) <= 3
            tm, tn, tk = (int(x) for x in f[f.index("tile") + 1].split("x"))
            cfg = (int(f[f.index("cluster") + 1]), tm, tn, tk, int(f[f.index("stages") + 1]), int(f[f.index("raster") + 1]))
            assert cfg in have, l
        elif op == "skinny":
            assert int(f[f.index("grid") + 1]) >= 1 and int(f[f.index("kps") + 1]) in (1, 2, 4)
        else:
            assert int(f[f.index("persistent") + 1]) in (0, 1)
    assert any(l.startswith("matmul bf16 8192 8192 8192 0 0 ") for l in lines)


def test_the_search_space_covers_tile_cluster_stage_and_k_block_axes():
    """Tile N, cluster shape, ring depth and K-block width vary independently of one another."""
    import habu_b200
    cfgs = habu_b200.matmul_configs()
    assert {c.cluster for c in cfgs} == {1, 2}
    assert {c.tile_k for c in cfgs} == {64, 128}
    for cluster, tile_n in ((1, 256), (1, 128), (1, 64), (2, 256), (2, 128)):
        same_tile = [c for c in cfgs if c.cluster == cluster and c.tile_n == tile_n and c.tile_k == 64]
        assert len({c.stages for c in same_tile}) >= 2, (cluster, tile_n)     # the ring depth is its own axis
        assert len({c.raster_group for c in same_tile}) >= 3
    assert len({(c.cluster, c.tile_n, c.tile_k, c.stages, c.raster_group) for c in cfgs}) == len(cfgs)


@pytest.mark.gpu
def test_search_then_cached_and_file_round_trip(ctx, tmp_path):
    import habu_b200 as hb
    r = ctx.autotune(512, 768, 256, search=True)
    assert 0 <= r.config_id < len(hb.matmul_configs()) and r.ms > 0
    c = ctx.autotune(512, 768, 256, search=False)
    assert c.config_id == r.config_id
    # M <= 64 goes to the stream-K kernel: the search is over its grid and k-blocks per stage
    sk = ctx.autotune(16, 2048, 2048, search=True)
    assert sk.config_id == -1 and 1 <= sk.split_k <= ctx.sm_count and sk.tile_k in (64, 128, 256) and sk.ms > 0
    # attention: one unit per CTA or the persistent work queue
    at = ctx.autotune_attention(2, 1024, 8, 2, causal=True, search=True)
    assert at.config_id in (0, 1) and at.ms > 0
    path = str(tmp_path / "cache.txt")
    ctx.tune_cache_save(path)
    text = open(path).read()
    assert text.startswith("# habu_b200 autotune cache v2")
    assert "matmul bf16 512 768 256 0 0 sm" in text and " = cluster " in text
    assert "skinny bf16 16 2048 2048 0 0 sm" in text and " = grid " in text
    assert "attention bf16 2 1024 128 1 " in text and " = persistent " in text
    other = hb.Context(0, load_tune_cache=False)
    with pytest.raises(hb.HabuError) as e:
        other.autotune(512, 768, 256, search=False)
    assert e.value.status == 2                  # `Not_found
    other.tune_cache_load(path)
    assert other.autotune(512, 768, 256, search=False).config_id == r.config_id
    again = other.autotune(16, 2048, 2048, search=False)
    assert (again.split_k, again.tile_k) == (sk.split_k, sk.tile_k)
    assert other.autotune_attention(2, 1024, 8, 2, causal=True, search=False).config_id == at.config_id
    with pytest.raises(hb.HabuError):
        other.tune_cache_load(str(tmp_path / "missing.txt"))
    # a version-1 file (index-valued lines, no GPU name) is still read
    v1 = tmp_path / "v1.txt"
    v1.write_text("# habu_b200 autotune cache v1\nmatmul bf16 640 640 640 0 0 sm%d = 9 0.5\n" % ctx.sm_count)
    other.tune_cache_load(str(v1))
    got = other.autotune(640, 640, 640, search=False)
    assert (got.cluster, got.tile_n, got.stages, got.raster_group) == (2, 256, 6, 8)
    other.close()
