"""ctypes declarations for libhabu_b200.so (the C ABI in ``include/habu_b200.h``).

There is no fallback: if the shared library is missing or does not load, importing this
module raises, and every product call goes through these bindings.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhabu_b200.so")

HB_OK, HB_ERR_INVALID, HB_ERR_NOT_FOUND, HB_ERR_DUPLICATE, HB_ERR_CUDA, HB_ERR_NCCL, \
    HB_ERR_TIMEOUT, HB_ERR_UNSUPPORTED, HB_ERR_NOMEM = range(9)
STATUS_NAMES = ["OK", "Invalid", "Not_found", "Duplicate", "Cuda", "Nccl", "Timeout",
                "Unsupported", "No_memory"]
HB_F32, HB_BF16, HB_I32 = 0, 1, 2
HB_EPI_NONE, HB_EPI_GELU, HB_EPI_SWIGLU, HB_EPI_RESIDUAL = 0, 1, 2, 3
HB_AR_AUTO, HB_AR_NCCL, HB_AR_P2P, HB_AR_NVLS = 0, 1, 2, 3
HB_OP_MATMUL, HB_OP_ATTENTION = 0, 1
HB_MATMUL_WEIGHTS_B = 0x100
HB_TUNE_CACHED, HB_TUNE_SEARCH = 0, 1
HB_UNIQUE_ID_BYTES = 128
HB_IPC_HANDLE_BYTES = 64


class hb_tensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dtype", C.c_int32), ("rank", C.c_int32),
                ("shape", C.c_int64 * 4), ("stride", C.c_int64 * 4)]


class hb_matmul_opts(C.Structure):
    _fields_ = [("epilogue", C.c_int32), ("config_id", C.c_int32), ("residual", C.c_void_p),
                ("residual_ld", C.c_int64)]


class hb_attn_opts(C.Structure):
    _fields_ = [("causal", C.c_int32), ("scale", C.c_float), ("lse", C.c_void_p),
                ("config_id", C.c_int32)]


class hb_op_desc(C.Structure):
    _fields_ = [("op", C.c_int32), ("dtype", C.c_int32), ("m", C.c_int64), ("n", C.c_int64),
                ("k", C.c_int64), ("layout", C.c_int32), ("epilogue", C.c_int32)]


class hb_tune_result(C.Structure):
    _fields_ = [("config_id", C.c_int32), ("tile_m", C.c_int32), ("tile_n", C.c_int32),
                ("tile_k", C.c_int32), ("stages", C.c_int32), ("cluster", C.c_int32),
                ("raster_group", C.c_int32), ("split_k", C.c_int32), ("ms", C.c_float),
                ("tflops", C.c_float)]


class hb_matmul_route(C.Structure):
    _fields_ = [("kernel", C.c_int32), ("config_id", C.c_int32), ("grid", C.c_int32), ("tiles", C.c_int32),
                ("max_segments", C.c_int32), ("scratch_bytes", C.c_int64)]


class hb_node(C.Structure):
    _fields_ = [("kind", C.c_int32), ("inputs", C.c_int32 * 4), ("out", C.c_int32),
                ("iparam", C.c_int32 * 4), ("fparam", C.c_float * 2), ("stream", C.c_int32)]


def load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m habu_b200.build` "
            "(there is no CPU or library fallback)")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
    T = C.POINTER(hb_tensor)
    sigs = {
        "hb_ctx_create": [i32, C.POINTER(vp)],
        "hb_ctx_destroy": [vp],
        "hb_ctx_set_stream": [vp, vp],
        "hb_alloc": [vp, C.c_size_t, C.POINTER(vp)],
        "hb_free": [vp, vp],
        "hb_upload": [vp, vp, vp, C.c_size_t],
        "hb_download": [vp, vp, vp, C.c_size_t],
        "hb_sync": [vp],
        "hb_matmul": [vp, T, T, T, C.POINTER(hb_matmul_opts)],
        "hb_matmul_gathered": [vp, T, T, T, C.POINTER(hb_matmul_opts)],
        "hb_matmul_host": [vp, vp, vp, vp, i64, i64, i64, i32],
        "hb_matmul_skinny_static": [vp, vp, vp, i64, i64, i64, i32, vp],
        "hb_static_status": [i32, C.POINTER(i32)],
        "hb_attention": [vp, T, T, T, T, C.POINTER(hb_attn_opts)],
        "hb_attention_host": [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i32, f32],
        "hb_rope_append": [vp, vp, i64, vp, vp, i64, i64, i64, i64, i64, f32],
        "hb_attention_decode": [vp, vp, i64, vp, vp, vp, i64, i64, i64, i64, i64, i64, f32],
        "hb_advance_pos": [vp, vp, i32],
        "hb_rmsnorm": [vp, vp, vp, vp, vp, i64, i64, f32],
        "hb_rope": [vp, vp, i64, i64, i64, i64, i64, f32, i64],
        "hb_embedding": [vp, vp, vp, vp, i64, i64, i64],
        "hb_swiglu": [vp, vp, vp, i64, i64],
        "hb_gelu": [vp, vp, vp, i64],
        "hb_gelu_backward": [vp, vp, vp, vp, i64],
        "hb_add": [vp, vp, vp, vp, i64],
        "hb_argmax": [vp, vp, vp, i64, i64],
        "hb_mse": [vp, vp, vp, vp, vp, i64],
        "hb_adam_step": [vp, vp, vp, vp, vp, vp, i64, f32, f32, f32, f32, i64, f32],
        "hb_adam_step_async": [vp, vp, vp, vp, vp, vp, i64, f32, f32, f32, f32, i64, f32],
        "hb_comm_unique_id": [vp],
        "hb_comm_init_rank": [vp, i32, i32, vp],
        "hb_comm_destroy": [vp],
        "hb_p2p_alloc": [vp, C.c_size_t, C.POINTER(vp), vp],
        "hb_p2p_attach": [vp, i32, i32, vp, C.c_size_t],
        "hb_p2p_attach_external": [vp, i32, i32, C.POINTER(vp), vp, C.c_size_t],
        "hb_all_reduce": [vp, vp, i64, i32, i32],
        "hb_comm_set_wait_limit": [vp, C.c_uint32],
        "hb_comm_configure": [vp, i32, i32],
        "hb_all_reduce_async": [vp, vp, i64, i32, i32],
        "hb_side_join": [vp],
        "hb_all_reduce_norm": [vp, vp, vp, vp, vp, vp, i64, i64, f32, i32, i32],
        "hb_graph_create": [vp, C.POINTER(vp)],
        "hb_graph_destroy": [vp],
        "hb_graph_input": [vp, T, C.POINTER(i32)],
        "hb_graph_temp": [vp, i32, i32, C.POINTER(i64), i32, C.POINTER(i32)],
        "hb_graph_view": [vp, i32, i64, i32, C.POINTER(i64), C.POINTER(i64), C.POINTER(i32)],
        "hb_graph_add": [vp, C.POINTER(hb_node)],
        "hb_graph_plan": [vp, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)],
        "hb_plan_arena": [i32, C.POINTER(C.c_size_t), C.POINTER(i32), C.POINTER(i32), C.POINTER(C.c_size_t),
                          C.POINTER(C.c_size_t)],
        "hb_graph_run": [vp],
        "hb_graph_capture": [vp],
        "hb_graph_replay": [vp],
        "hb_graph_run_timed": [vp, C.POINTER(C.c_float), i32],
        "hb_graph_describe": [vp, C.c_char_p, C.c_size_t],
        "hb_graph_tensor_ptr": [vp, i32, C.POINTER(vp)],
        "hb_autotune": [vp, C.POINTER(hb_op_desc), i32, C.POINTER(hb_tune_result)],
        "hb_tune_cache_load": [vp, C.c_char_p],
        "hb_tune_cache_save": [vp, C.c_char_p],
        "hb_matmul_default_route": [i32, C.POINTER(hb_op_desc), C.POINTER(hb_matmul_route)],
        "hb_matmul_config_info": [i32, C.POINTER(hb_tune_result)],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = i32
    lib.hb_last_error_string.argtypes = [vp]
    lib.hb_last_error_string.restype = C.c_char_p
    lib.hb_static_last_error.argtypes = []
    lib.hb_static_last_error.restype = C.c_char_p
    lib.hb_p2p_flag_bytes.argtypes = []
    lib.hb_p2p_flag_bytes.restype = C.c_size_t
    lib.hb_launch_count.argtypes = [vp]
    lib.hb_launch_count.restype = i64
    lib.hb_sm_count.argtypes = [vp]
    lib.hb_sm_count.restype = i32
    lib.hb_matmul_config_count.argtypes = []
    lib.hb_matmul_config_count.restype = i32
    return lib
