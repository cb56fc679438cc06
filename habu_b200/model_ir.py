"""Host-side mirror of the model-IR operator surface over the C ABI.

The reference project has no operator interface for this path (its ``src/lib`` holds a
SLEIGH parser only), so the names follow the operator list the executor is specified
with: ``matmul``, ``attention``, ``all_reduce`` nodes and the ``autotune`` entry point.
Its conventions are kept where they apply: constructors validate and errors are values
(``src/lib/error.ml:18-26``) -- surfaced here as :class:`HabuError` carrying the status
code, never as a silent fallback.

Everything runs on the GPU through ``libhabu_b200.so``; numpy arrays appear only as
host-side sources and destinations of explicit uploads and downloads.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from . import _capi
from ._capi import (HB_AR_AUTO, HB_AR_NCCL, HB_AR_NVLS, HB_AR_P2P, HB_BF16, HB_EPI_GELU, HB_EPI_NONE,
                    HB_EPI_RESIDUAL, HB_EPI_SWIGLU, HB_F32, HB_I32, HB_OP_MATMUL,
                    HB_TUNE_CACHED, HB_TUNE_SEARCH)

_lib = _capi.load()
_ELEM = {HB_F32: 4, HB_BF16: 2, HB_I32: 4}


class HabuError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"`{_capi.STATUS_NAMES[status]}: {message}")
        self.status = status


@dataclass
class Tensor:
    """A device tensor view: pointer, dtype, shape and strides (in elements)."""
    ptr: int
    dtype: int
    shape: tuple
    stride: tuple
    owner: object = None

    @property
    def nbytes(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n * _ELEM[self.dtype]

    @property
    def T(self) -> "Tensor":
        assert len(self.shape) == 2
        return Tensor(self.ptr, self.dtype, self.shape[::-1], self.stride[::-1], self.owner)

    def c(self) -> _capi.hb_tensor:
        t = _capi.hb_tensor()
        t.ptr = self.ptr
        t.dtype = self.dtype
        t.rank = len(self.shape)
        for i, (s, st) in enumerate(zip(self.shape, self.stride)):
            t.shape[i] = s
            t.stride[i] = st
        return t


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Host-side fp32 -> bf16 bit patterns, round to nearest even (NaNs stay NaNs)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    rounded = (u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    return np.where(nan, (u >> np.uint32(16)) | np.uint32(0x40), rounded).astype(np.uint16)


def _contig(shape) -> tuple:
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= s
    return tuple(reversed(st))


class Context:
    """One context per GPU (and per host thread or process)."""

    def __init__(self, device: int = 0, load_tune_cache: bool = True):
        h = C.c_void_p()
        st = _lib.hb_ctx_create(device, C.byref(h))
        if st != 0:
            raise HabuError(st, f"hb_ctx_create(device={device}) failed; an sm_100 GPU is required")
        self._h = h
        self.device = device
        import os
        cache = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tune_cache.txt")
        if load_tune_cache and os.path.exists(cache):     # persisted autotune choices
            self.tune_cache_load(cache)

    # -- plumbing ---------------------------------------------------------------
    def _check(self, st: int):
        if st != 0:
            raise HabuError(st, _lib.hb_last_error_string(self._h).decode())

    def close(self):
        if self._h:
            _lib.hb_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_stream(self, cuda_stream: Optional[int]):
        self._check(_lib.hb_ctx_set_stream(self._h, C.c_void_p(cuda_stream)))

    def sync(self):
        self._check(_lib.hb_sync(self._h))

    @property
    def launches(self) -> int:
        return int(_lib.hb_launch_count(self._h))

    @property
    def sm_count(self) -> int:
        return int(_lib.hb_sm_count(self._h))

    # -- memory -----------------------------------------------------------------
    def empty(self, shape: Sequence[int], dtype: int = HB_BF16) -> Tensor:
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        p = C.c_void_p()
        self._check(_lib.hb_alloc(self._h, n * _ELEM[dtype], C.byref(p)))
        return Tensor(p.value, dtype, shape, _contig(shape))

    def free(self, t: Tensor):
        self._check(_lib.hb_free(self._h, C.c_void_p(t.ptr)))

    def wrap(self, ptr: int, shape, dtype=HB_BF16, stride=None, owner=None) -> Tensor:
        shape = tuple(int(s) for s in shape)
        return Tensor(int(ptr), dtype, shape, tuple(stride) if stride else _contig(shape), owner)

    def upload(self, host: np.ndarray, dtype: Optional[int] = None) -> Tensor:
        """Copy a C-contiguous host array to a new device tensor.  uint16 arrays are
        bf16 bit patterns, float32 -> HB_F32, int32 -> HB_I32."""
        host = np.ascontiguousarray(host)
        if dtype is None:
            dtype = {np.dtype(np.uint16): HB_BF16, np.dtype(np.float32): HB_F32,
                     np.dtype(np.int32): HB_I32}[host.dtype]
        t = self.empty(host.shape, dtype)
        self._check(_lib.hb_upload(self._h, C.c_void_p(t.ptr), host.ctypes.data_as(C.c_void_p), host.nbytes))
        self.sync()
        return t

    def download(self, t: Tensor) -> np.ndarray:
        np_dtype = {HB_BF16: np.uint16, HB_F32: np.float32, HB_I32: np.int32}[t.dtype]
        assert t.stride == _contig(t.shape), "download needs a contiguous tensor"
        out = np.empty(t.shape, np_dtype)
        self._check(_lib.hb_download(self._h, out.ctypes.data_as(C.c_void_p), C.c_void_p(t.ptr), out.nbytes))
        self.sync()
        return out

    # -- matmul node --------------------------------------------------------------
    def matmul(self, A: Tensor, B: Tensor, out: Optional[Tensor] = None, epilogue: int = HB_EPI_NONE,
               residual: Optional[Tensor] = None, config_id: int = -1, weights: bool = False) -> Tensor:
        """out[M,N] = epilogue(A[M,K] @ B[K,N]); layouts are read from the strides.  `weights`:
        B is a weight matrix that nothing in flight writes (lets the M <= 64 kernel stream it in
        while the kernel in front is still running)."""
        M, N = A.shape[0], B.shape[1]
        if out is None:
            out = self.empty((M, N // 2 if epilogue == HB_EPI_SWIGLU else N), A.dtype)
        opts = _capi.hb_matmul_opts(epilogue | (_capi.HB_MATMUL_WEIGHTS_B if weights else 0), config_id,
                                    residual.ptr if residual else None, residual.stride[0] if residual else 0)
        ta, tb, tc = A.c(), B.c(), out.c()
        self._check(_lib.hb_matmul(self._h, C.byref(ta), C.byref(tb), C.byref(tc), C.byref(opts)))
        return out

    def matmul_host(self, A: np.ndarray, Bt: np.ndarray, dtype: int = HB_BF16) -> np.ndarray:
        """Host-buffer call: A [M,K] row-major, Bt [N,K] (B column-major); returns C [M,N]."""
        M, K = A.shape
        N = Bt.shape[0]
        out = np.empty((M, N), A.dtype)
        self._check(_lib.hb_matmul_host(self._h, A.ctypes.data_as(C.c_void_p), Bt.ctypes.data_as(C.c_void_p),
                                        out.ctypes.data_as(C.c_void_p), M, N, K, dtype))
        return out

    # -- attention node -----------------------------------------------------------
    def attention(self, Q: Tensor, K: Tensor, V: Tensor, out: Optional[Tensor] = None, causal: bool = True,
                  scale: Optional[float] = None, lse: Optional[Tensor] = None) -> Tensor:
        """Q [B,S,Hq,D], K/V [B,S,Hkv,D] -> O [B,S,Hq,D]."""
        if out is None:
            out = self.empty(Q.shape, Q.dtype)
        if scale is None:
            scale = float(Q.shape[-1]) ** -0.5
        opts = _capi.hb_attn_opts(int(causal), scale, lse.ptr if lse else None, -1)
        tq, tk, tv, to = Q.c(), K.c(), V.c(), out.c()
        self._check(_lib.hb_attention(self._h, C.byref(tq), C.byref(tk), C.byref(tv), C.byref(to), C.byref(opts)))
        return out

    def attention_host(self, Q: np.ndarray, K: np.ndarray, V: np.ndarray, causal=True, scale=None) -> np.ndarray:
        B, S, Hq, D = Q.shape
        Hkv = K.shape[2]
        if scale is None:
            scale = float(D) ** -0.5
        out = np.empty_like(Q)
        self._check(_lib.hb_attention_host(
            self._h, Q.ctypes.data_as(C.c_void_p), K.ctypes.data_as(C.c_void_p), V.ctypes.data_as(C.c_void_p),
            out.ctypes.data_as(C.c_void_p), B, S, Hq, Hkv, D, int(causal), scale))
        return out

    # -- decode-shaped path ----------------------------------------------------------
    def rope_append(self, qkv: Tensor, kv_cache: Tensor, pos: Tensor, n_q_heads: int, n_kv_heads: int,
                    base: float = 10000.0):
        """RoPE of the new token's q and k heads at position pos[0] (in place in `qkv`
        [batch, row]) and append of k and v to `kv_cache` [2*batch, s_max, kv_heads, 128]."""
        self._check(_lib.hb_rope_append(self._h, qkv.ptr, qkv.stride[0], kv_cache.ptr, pos.ptr, qkv.shape[0], n_q_heads,
                                        n_kv_heads, kv_cache.shape[3], kv_cache.shape[1], base))

    def attention_decode(self, qkv: Tensor, kv_cache: Tensor, pos: Tensor, n_q_heads: int, n_kv_heads: int,
                         out: Optional[Tensor] = None, scale: Optional[float] = None, len_hint: int = 0) -> Tensor:
        """Single-query attention of each sequence's new token over cache positions 0..pos[0]."""
        D = kv_cache.shape[3]
        if out is None:
            out = self.empty((qkv.shape[0], n_q_heads * D))
        if scale is None:
            scale = float(D) ** -0.5
        self._check(_lib.hb_attention_decode(self._h, qkv.ptr, qkv.stride[0], kv_cache.ptr, pos.ptr, out.ptr, qkv.shape[0],
                                             n_q_heads, n_kv_heads, D, kv_cache.shape[1], len_hint, scale))
        return out

    def advance_pos(self, pos: Tensor, n: int = 1):
        self._check(_lib.hb_advance_pos(self._h, pos.ptr, n))

    # -- glue ---------------------------------------------------------------------
    def rmsnorm(self, x: Tensor, gain: Tensor, out: Optional[Tensor] = None, eps: float = 1e-5,
                residual: Optional[Tensor] = None) -> Tensor:
        rows, cols = x.shape
        if out is None:
            out = self.empty(x.shape, x.dtype)
        self._check(_lib.hb_rmsnorm(self._h, x.ptr, gain.ptr, out.ptr, residual.ptr if residual else None,
                                    rows, cols, eps))
        return out

    def rope(self, x: Tensor, seq: int, heads: int, head_dim: int, base: float = 10000.0, pos0: int = 0) -> Tensor:
        tokens = x.shape[0]
        self._check(_lib.hb_rope(self._h, x.ptr, tokens, seq, heads, head_dim, x.stride[0], base, pos0))
        return x

    def embedding(self, table: Tensor, ids: Tensor, out: Optional[Tensor] = None) -> Tensor:
        tokens = ids.shape[0]
        vocab, dim = table.shape
        if out is None:
            out = self.empty((tokens, dim), table.dtype)
        self._check(_lib.hb_embedding(self._h, table.ptr, ids.ptr, out.ptr, tokens, vocab, dim))
        return out

    def swiglu(self, x: Tensor, out: Optional[Tensor] = None) -> Tensor:
        rows, two = x.shape
        if out is None:
            out = self.empty((rows, two // 2), x.dtype)
        self._check(_lib.hb_swiglu(self._h, x.ptr, out.ptr, rows, two // 2))
        return out

    def gelu(self, x: Tensor, out: Optional[Tensor] = None) -> Tensor:
        if out is None:
            out = self.empty(x.shape, x.dtype)
        self._check(_lib.hb_gelu(self._h, x.ptr, out.ptr, x.nbytes // 2))
        return out

    def gelu_backward(self, x: Tensor, dy: Tensor, out: Optional[Tensor] = None) -> Tensor:
        if out is None:
            out = self.empty(x.shape, x.dtype)
        self._check(_lib.hb_gelu_backward(self._h, x.ptr, dy.ptr, out.ptr, x.nbytes // 2))
        return out

    def add(self, a: Tensor, b: Tensor, out: Optional[Tensor] = None) -> Tensor:
        if out is None:
            out = self.empty(a.shape, a.dtype)
        self._check(_lib.hb_add(self._h, a.ptr, b.ptr, out.ptr, a.nbytes // 2))
        return out

    def mse(self, y: Tensor, target: Tensor, dy: Optional[Tensor] = None, loss: Optional[Tensor] = None):
        """Returns (loss tensor f32[1], dy) for mean((y - target)^2)."""
        if dy is None:
            dy = self.empty(y.shape, y.dtype)
        if loss is None:
            loss = self.empty((1,), HB_F32)
        self._check(_lib.hb_mse(self._h, y.ptr, target.ptr, dy.ptr, loss.ptr, y.nbytes // 2))
        return loss, dy

    def adam_step(self, w: Tensor, m: Tensor, v: Tensor, grad: Tensor, w_bf16: Tensor, step: int, lr=1e-3, beta1=0.9,
                  beta2=0.999, eps=1e-8, grad_scale=1.0, on_side_stream: bool = False):
        """on_side_stream: enqueue the update on the side stream behind everything queued so far
        (pair with side_join()), so that it runs under the products that follow."""
        fn = _lib.hb_adam_step_async if on_side_stream else _lib.hb_adam_step
        self._check(fn(self._h, w.ptr, m.ptr, v.ptr, grad.ptr, w_bf16.ptr, w.nbytes // 4, lr, beta1, beta2, eps, step,
                       grad_scale))

    def argmax(self, x: Tensor) -> Tensor:
        rows, cols = x.shape
        out = self.empty((rows,), HB_I32)
        self._check(_lib.hb_argmax(self._h, x.ptr, out.ptr, rows, cols))
        return out

    # -- collective node ------------------------------------------------------------
    @staticmethod
    def comm_unique_id() -> bytes:
        buf = C.create_string_buffer(_capi.HB_UNIQUE_ID_BYTES)
        st = _lib.hb_comm_unique_id(buf)
        if st != 0:
            raise HabuError(st, "hb_comm_unique_id failed")
        return buf.raw

    def comm_init_rank(self, world: int, rank: int, unique_id: bytes):
        self._check(_lib.hb_comm_init_rank(self._h, world, rank, unique_id))

    def p2p_alloc(self, nbytes: int):
        p = C.c_void_p()
        handle = C.create_string_buffer(_capi.HB_IPC_HANDLE_BYTES)
        self._check(_lib.hb_p2p_alloc(self._h, nbytes, C.byref(p), handle))
        return p.value, handle.raw

    def p2p_attach(self, world: int, rank: int, handles: Sequence[bytes], nbytes: int):
        self._check(_lib.hb_p2p_attach(self._h, world, rank, b"".join(handles), nbytes))

    @staticmethod
    def p2p_flag_bytes() -> int:
        return int(_lib.hb_p2p_flag_bytes())

    def p2p_attach_external(self, world: int, rank: int, peer_ptrs: Sequence[int], multicast_ptr: Optional[int],
                            nbytes: int):
        """Register a caller-owned symmetric buffer (and its multicast mapping, if any)."""
        arr = (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in peer_ptrs])
        self._check(_lib.hb_p2p_attach_external(self._h, world, rank, arr, C.c_void_p(multicast_ptr or 0), nbytes))

    def comm_configure(self, fused_form: int = 0, fused_ctas: int = 0):
        """Kernel form of the fused collective: 0 automatic, 1 CTA per row, 2 warp per row on at
        most `fused_ctas` CTAs (the form that runs beside a GEMM)."""
        self._check(_lib.hb_comm_configure(self._h, fused_form, fused_ctas))

    def comm_set_wait_limit(self, polls: int):
        """Polls per cross-GPU flag wait before a collective kernel reports HB_ERR_TIMEOUT."""
        self._check(_lib.hb_comm_set_wait_limit(self._h, polls))

    def all_reduce(self, x: Tensor, algo: int = HB_AR_AUTO) -> Tensor:
        n = 1
        for s in x.shape:
            n *= s
        self._check(_lib.hb_all_reduce(self._h, x.ptr, n, x.dtype, algo))
        return x

    def all_reduce_async(self, x: Tensor, algo: int = HB_AR_AUTO) -> Tensor:
        """The allreduce on the side stream (after everything queued so far); pair with side_join()."""
        n = 1
        for s in x.shape:
            n *= s
        self._check(_lib.hb_all_reduce_async(self._h, x.ptr, n, x.dtype, algo))
        return x

    def side_join(self):
        self._check(_lib.hb_side_join(self._h))

    # -- autotune entry point ---------------------------------------------------------
    def autotune(self, m: int, n: int, k: int, layout: int = 0, epilogue: int = HB_EPI_NONE,
                 search: bool = True) -> _capi.hb_tune_result:
        d = _capi.hb_op_desc(HB_OP_MATMUL, HB_BF16, m, n, k, layout, epilogue)
        r = _capi.hb_tune_result()
        self._check(_lib.hb_autotune(self._h, C.byref(d), HB_TUNE_SEARCH if search else HB_TUNE_CACHED, C.byref(r)))
        return r

    def autotune_attention(self, batch: int, seq: int, n_q_heads: int, n_kv_heads: int, causal: bool = True,
                           search: bool = True) -> _capi.hb_tune_result:
        """Attention node: one work unit per CTA (config 0) against the persistent work queue (1)."""
        d = _capi.hb_op_desc(_capi.HB_OP_ATTENTION, HB_BF16, batch, seq, 128, int(causal), (n_q_heads << 16) | n_kv_heads)
        r = _capi.hb_tune_result()
        self._check(_lib.hb_autotune(self._h, C.byref(d), HB_TUNE_SEARCH if search else HB_TUNE_CACHED, C.byref(r)))
        return r

    def tune_cache_save(self, path: str):
        self._check(_lib.hb_tune_cache_save(self._h, path.encode()))

    def tune_cache_load(self, path: str):
        self._check(_lib.hb_tune_cache_load(self._h, path.encode()))


def matmul_configs():
    out = []
    for i in range(_lib.hb_matmul_config_count()):
        r = _capi.hb_tune_result()
        _lib.hb_matmul_config_info(i, C.byref(r))
        out.append(r)
    return out


def matmul_default_route(m: int, n: int, k: int, layout: int = 0, epilogue: int = HB_EPI_NONE, sm_count: int = 148):
    """Kernel and configuration the dispatcher picks for a bf16 matmul that has no autotune
    cache entry (``hb_matmul_default_route``; host arithmetic, needs no GPU)."""
    d = _capi.hb_op_desc(0, HB_BF16, m, n, k, layout, epilogue)
    r = _capi.hb_matmul_route()
    st = _lib.hb_matmul_default_route(sm_count, C.byref(d), C.byref(r))
    if st != 0:
        raise ValueError(f"hb_matmul_default_route: status {st}")
    return r
