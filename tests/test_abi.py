"""The C-ABI library loads and exports every symbol the public header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "habu_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_operator_surface():
    syms = declared_symbols()
    for name in ["hb_matmul", "hb_attention", "hb_all_reduce", "hb_autotune", "hb_ctx_create", "hb_sync"]:
        assert name in syms


def test_library_exports_every_declared_symbol():
    from habu_b200 import _capi
    lib = ctypes.CDLL(_capi.LIB_PATH)
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_binding_covers_every_declared_symbol():
    from habu_b200 import _capi
    lib = _capi.load()
    for s in declared_symbols():
        fn = getattr(lib, s)
        assert fn.argtypes is not None, f"{s} has no ctypes signature"


def test_config_table_is_described_without_a_gpu():
    import habu_b200
    cfgs = habu_b200.matmul_configs()
    assert len(cfgs) >= 3
    assert all(c.tile_m in (128, 256) and c.tile_k in (64, 128) and c.stages >= 2 for c in cfgs)


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "habu_b200")
    for name in os.listdir(pkg):
        if name.endswith(".py"):
            text = open(os.path.join(pkg, name)).read()
            assert not re.search(r"^\s*(import|from)\s+oracle\b", text, flags=re.M), name


def test_host_bf16_conversion_matches_the_oracle_bit_for_bit():
    import numpy as np

    import oracle
    from habu_b200.model_ir import f32_to_bf16_bits
    x = oracle.normal((50000,), 3, 0.0, 5.0)
    x[:9] = [0.0, -0.0, np.inf, -np.inf, np.nan, 1.00390625, 1.01171875, 3.0e38, 1e-40]
    assert np.array_equal(f32_to_bf16_bits(x), oracle.to_bf16_bits(x))


def test_static_entry_points_refuse_a_device_that_is_not_current():
    """No GPU needed: with no current device (or another one) the look-up of the static
    arrays must be refused, never cached under the wrong index."""
    from habu_b200 import _capi
    lib = _capi.load()
    words = (ctypes.c_int32 * 4)()
    assert lib.hb_static_status(63, words) == 1
    assert b"current CUDA device" in lib.hb_static_last_error()
    assert lib.hb_static_status(-1, words) == 1


def test_host_buffer_placement_helpers(tmp_path):
    """sysfs parsing of the pinned-buffer placement helper, against a fake sysfs tree."""
    from habu_b200 import hostmem
    assert hostmem.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert hostmem.parse_cpulist("") == []
    assert hostmem.normalise_bus_id("00000000:1B:00.0") == "0000:1b:00.0"
    assert hostmem.normalise_bus_id("1b:00.0") == "0000:1b:00.0"
    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node"
    node.mkdir(parents=True)
    (node / "online").write_text("0-1\n")
    assert hostmem.gpu_numa_node("0000:1B:00.0", str(tmp_path)) == 1
    assert hostmem.gpu_numa_node("0000:1c:00.0", str(tmp_path)) is None
    (dev / "numa_node").write_text("-1\n")
    assert hostmem.gpu_numa_node("0000:1b:00.0", str(tmp_path)) is None
    assert hostmem.online_nodes(str(tmp_path)) == [0, 1]
    # no answer from sysfs: the block runs unchanged and says so
    with hostmem.near_gpu("0000:1b:00.0", str(tmp_path)) as place:
        pass
    assert place.outcome.startswith("unchanged")
    with hostmem.near_gpu(None) as place:
        pass
    assert place.outcome.startswith("unchanged")


def test_host_buffer_placement_sets_and_restores_policy(tmp_path, monkeypatch):
    """With a GPU on node 1 of a two-node box the block asks for MPOL_PREFERRED on node 1 and
    puts the default policy back on exit; a refused call leaves everything unchanged."""
    from habu_b200 import hostmem
    dev = tmp_path / "bus/pci/devices/0000:9a:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node"
    node.mkdir(parents=True)
    (node / "online").write_text("0-1\n")
    calls = []
    monkeypatch.setattr(hostmem, "_set_mempolicy", lambda mode, n: calls.append((mode, n)) or 0)
    with hostmem.near_gpu("0000:9A:00.0", str(tmp_path)) as place:
        assert calls == [(hostmem._MPOL_PREFERRED, 1)]
    assert place.outcome == "preferred" and place.node == 1
    assert calls[-1] == (hostmem._MPOL_DEFAULT, None)
    calls.clear()
    monkeypatch.setattr(hostmem, "_set_mempolicy", lambda mode, n: calls.append((mode, n)) or -1)
    with hostmem.near_gpu("0000:9a:00.0", str(tmp_path)) as place:
        pass
    assert place.outcome.startswith("unchanged: set_mempolicy refused") and len(calls) == 1
