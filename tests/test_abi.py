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
