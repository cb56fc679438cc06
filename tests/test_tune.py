"""Autotune cache: the persisted text format round-trips (no GPU needed for the file
checks), and on a GPU a search records a winner that the cached mode then returns."""
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CACHE = os.path.join(ROOT, "habu_b200", "tune_cache.txt")


def test_committed_cache_is_well_formed():
    lines = [l for l in open(CACHE).read().splitlines() if l and not l.startswith("#")]
    assert len(lines) >= 10
    import habu_b200
    n_cfg = len(habu_b200.matmul_configs())
    for l in lines:
        key, val = l.split(" = ")
        op, dtype, m, n, k, layout, epi, sm = key.split()
        assert op == "matmul" and dtype == "bf16" and sm.startswith("sm")
        assert all(int(x) > 0 for x in (m, n, k)) and 0 <= int(layout) <= 3 and 0 <= int(epi) <= 3
        cfg, ms = val.split()
        assert 0 <= int(cfg) < n_cfg and float(ms) > 0
    assert any(l.startswith("matmul bf16 8192 8192 8192 0 0 ") for l in lines)


@pytest.mark.gpu
def test_search_then_cached_and_file_round_trip(ctx, tmp_path):
    import habu_b200 as hb
    r = ctx.autotune(512, 768, 256, search=True)
    assert 0 <= r.config_id < len(hb.matmul_configs()) and r.ms > 0
    c = ctx.autotune(512, 768, 256, search=False)
    assert c.config_id == r.config_id
    path = str(tmp_path / "cache.txt")
    ctx.tune_cache_save(path)
    text = open(path).read()
    assert "matmul bf16 512 768 256 0 0 sm" in text
    other = hb.Context(0, load_tune_cache=False)
    with pytest.raises(hb.HabuError) as e:
        other.autotune(512, 768, 256, search=False)
    assert e.value.status == 2                  # `Not_found
    other.tune_cache_load(path)
    assert other.autotune(512, 768, 256, search=False).config_id == r.config_id
    with pytest.raises(hb.HabuError):
        other.tune_cache_load(str(tmp_path / "missing.txt"))
    other.close()
