"""habu_b200: sm_100a kernel library for the model-IR executor's dense hot path
(matmul, fused causal attention, tensor-parallel allreduce, autotune), reached through
the C ABI in ``include/habu_b200.h``.

The operator surface lives in :mod:`habu_b200.model_ir`, which loads
``libhabu_b200.so`` on first use and raises if it is missing or stale -- there is no CPU
or library fallback.  ``python -m habu_b200.build`` compiles the library in-tree.
"""
_EXPORTS = ["Context", "HabuError", "Tensor", "matmul_configs", "HB_BF16", "HB_F32", "HB_I32", "HB_EPI_NONE",
            "HB_EPI_GELU", "HB_EPI_SWIGLU", "HB_EPI_RESIDUAL", "HB_AR_AUTO", "HB_AR_NCCL", "HB_AR_P2P", "HB_AR_NVLS"]
__all__ = list(_EXPORTS)


def __getattr__(name):
    if name in _EXPORTS or name in ("model_ir", "graph", "tp"):
        import importlib
        if name in ("model_ir", "graph", "tp"):
            return importlib.import_module(f".{name}", __name__)
        return getattr(importlib.import_module(".model_ir", __name__), name)
    raise AttributeError(name)
