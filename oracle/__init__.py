"""ctypes binding of the CPU checker (``oracle/hb_oracle.c``).

Test infrastructure only: imported by ``tests/``, ``__graft_entry__.smoke()`` and the
CPU-baseline / reference legs of ``bench.py``; the product package never imports it.
All arrays are C-contiguous float32 numpy arrays unless stated.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libhb_oracle.so")


def build() -> str:
    subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _SO


def _load():
    src = os.path.join(_HERE, "hb_oracle.c")
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        build()
    return C.CDLL(_SO)


def _bind(lib):
    lib.orc_mse.restype = C.c_double
    lib.orc_num_threads.restype = C.c_int
    return lib


_lib = _bind(_load())
_fp = C.POINTER(C.c_float)
_i64 = C.c_int64
_native = False


def use_native_build() -> bool:
    """For the timed CPU legs of ``bench.py`` only: rebuild the checker with ``-march=native``
    on the host it is about to be timed on (AVX-512 where the host has it) and switch this
    module to that build.  The portable x86-64-v3 build stays the one the tests use, so the
    golden fixtures do not depend on the host's vector width.  Returns False, leaving the
    portable build in place, when the host has no compiler or the build fails."""
    global _lib, _native
    if _native:
        return True
    so = os.path.join(_HERE, "libhb_oracle_native.so")
    try:
        subprocess.run(["make", "-C", _HERE, "-s", "-B", "libhb_oracle_native.so"], check=True,
                       stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, timeout=300)
        lib = _bind(C.CDLL(so))
        lib.orc_set_num_threads(C.c_int(num_threads()))
    except Exception:
        return False
    _lib, _native = lib, True
    return True


def is_native_build() -> bool:
    return _native


def _f(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(_fp)


def num_threads() -> int:
    return int(_lib.orc_num_threads())


def use_all_cores() -> int:
    """Let the checker use every core this process may run on (torchrun pins
    OMP_NUM_THREADS=1 for its workers); returns the thread count now in use."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    _lib.orc_set_num_threads(C.c_int(n))
    return num_threads()


def set_num_threads(n: int) -> int:
    """Use `n` threads (at least one); returns the thread count now in use."""
    _lib.orc_set_num_threads(C.c_int(max(1, int(n))))
    return num_threads()


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round fp32 values to bf16 (nearest-even) in place; returns x."""
    _lib.orc_round_bf16(_f(x), _i64(x.size))
    return x


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    y = np.empty(x.shape, np.uint16)
    _lib.orc_f32_to_bf16(_f(np.ascontiguousarray(x, np.float32)), y.ctypes.data_as(C.c_void_p), _i64(x.size))
    return y


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, np.uint16)
    y = np.empty(b.shape, np.float32)
    _lib.orc_bf16_to_f32(b.ctypes.data_as(C.c_void_p), _f(y), _i64(b.size))
    return y


def uniform(shape, seed: int, lo=-1.0, hi=1.0, offset=0) -> np.ndarray:
    x = np.empty(shape, np.float32)
    _lib.orc_fill_uniform(_f(x), _i64(x.size), C.c_uint64(seed), _i64(offset), C.c_float(lo), C.c_float(hi))
    return x


def normal(shape, seed: int, mean=0.0, std=1.0, offset=0) -> np.ndarray:
    x = np.empty(shape, np.float32)
    _lib.orc_fill_normal(_f(x), _i64(x.size), C.c_uint64(seed), _i64(offset), C.c_float(mean), C.c_float(std))
    return x


def gemm(A: np.ndarray, B: np.ndarray, acc_double: bool = False) -> np.ndarray:
    """C = A @ B for 2-D fp32 arrays of any (positive) strides."""
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    Cm = np.empty((M, N), np.float32)
    es = 4
    _lib.orc_gemm(A.ctypes.data_as(_fp), B.ctypes.data_as(_fp), _f(Cm), _i64(M), _i64(N), _i64(K),
                  _i64(A.strides[0] // es), _i64(A.strides[1] // es), _i64(B.strides[0] // es),
                  _i64(B.strides[1] // es), _i64(N), C.c_int(int(acc_double)))
    return Cm


def attention(Q, K, V, causal=True, scale=None, round_p=False, return_lse=False):
    """Q [B,S,Hq,D], K/V [B,S,Hkv,D] -> O [B,S,Hq,D] (and lse [B,Hq,S])."""
    B, S, Hq, D = Q.shape
    Hkv = K.shape[2]
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    O = np.empty_like(Q)
    lse = np.empty((B, Hq, S), np.float32)
    _lib.orc_attention(_f(Q), _f(K), _f(V), _f(O), _f(lse), _i64(B), _i64(S), _i64(Hq), _i64(Hkv),
                       _i64(D), C.c_int(int(causal)), C.c_float(scale), C.c_int(int(round_p)))
    return (O, lse) if return_lse else O


def rmsnorm(x, gain, eps=1e-5):
    y = np.empty_like(x)
    rows, cols = x.shape
    _lib.orc_rmsnorm(_f(x), _f(gain), _f(y), _i64(rows), _i64(cols), C.c_float(eps))
    return y


def rope(x, seq, heads, head_dim, base=10000.0, pos0=0):
    """x [tokens, heads*head_dim] (copied); returns the rotated copy."""
    y = np.ascontiguousarray(x, np.float32).copy()
    tokens = y.shape[0]
    _lib.orc_rope(_f(y), _i64(tokens), _i64(seq), _i64(heads), _i64(head_dim), _i64(y.shape[1]),
                  C.c_float(base), _i64(pos0))
    return y


def swiglu(x, interleaved=False):
    rows, two = x.shape
    out = np.empty((rows, two // 2), np.float32)
    fn = _lib.orc_swiglu_interleaved if interleaved else _lib.orc_swiglu
    fn(_f(x), _f(out), _i64(rows), _i64(two // 2))
    return out


def gelu(x):
    y = np.empty_like(x)
    _lib.orc_gelu(_f(x), _f(y), _i64(x.size))
    return y


def gelu_backward(x, dy):
    dx = np.empty_like(x)
    _lib.orc_gelu_backward(_f(x), _f(dy), _f(dx), _i64(x.size))
    return dx


def add(a, b):
    out = np.empty_like(a)
    _lib.orc_add(_f(a), _f(b), _f(out), _i64(a.size))
    return out


def embedding(table, ids):
    ids = np.ascontiguousarray(ids, np.int32)
    out = np.empty((ids.size, table.shape[1]), np.float32)
    _lib.orc_embedding(_f(table), ids.ctypes.data_as(C.c_void_p), _f(out), _i64(ids.size), _i64(table.shape[1]))
    return out


def argmax(x):
    rows, cols = x.shape
    out = np.empty(rows, np.int32)
    _lib.orc_argmax(_f(x), out.ctypes.data_as(C.c_void_p), _i64(rows), _i64(cols))
    return out


def mse(y, t) -> float:
    return float(_lib.orc_mse(_f(y), _f(t), _i64(y.size)))


def adam(w, m, v, g, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, step=1):
    """In-place Adam step on fp32 arrays w, m, v."""
    _lib.orc_adam(_f(w), _f(m), _f(v), _f(g), _i64(w.size), C.c_float(lr), C.c_float(b1), C.c_float(b2),
                  C.c_float(eps), _i64(step))


def all_reduce(bufs):
    """Sum-allreduce over a list of equal-size fp32 arrays, in place, rank order."""
    arr = (_fp * len(bufs))(*[_f(b) for b in bufs])
    _lib.orc_all_reduce(arr, C.c_int(len(bufs)), _i64(bufs[0].size))
