"""habu_b200: sm_100a kernel library for the model-IR executor's dense hot path
(matmul, fused causal attention, tensor-parallel allreduce, autotune), reached through
the C ABI in ``include/habu_b200.h``.  Importing the package loads ``libhabu_b200.so``
and raises if it is missing; no CPU or library fallback exists."""
from .model_ir import (Context, HabuError, Tensor, matmul_configs, HB_BF16, HB_F32, HB_I32, HB_EPI_NONE,
                       HB_EPI_GELU, HB_EPI_SWIGLU, HB_EPI_RESIDUAL, HB_AR_AUTO, HB_AR_NCCL, HB_AR_P2P)

__all__ = ["Context", "HabuError", "Tensor", "matmul_configs", "HB_BF16", "HB_F32", "HB_I32", "HB_EPI_NONE",
           "HB_EPI_GELU", "HB_EPI_SWIGLU", "HB_EPI_RESIDUAL", "HB_AR_AUTO", "HB_AR_NCCL", "HB_AR_P2P"]
