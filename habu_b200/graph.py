"""Host-side wrapper of the model-IR executor (``hb_graph_*`` in the C ABI): build an
ordered node list over tensor ids, let the library plan the arena, and run it."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

from . import _capi
from .model_ir import Context, Tensor, _contig, _lib

(NODE_MATMUL, NODE_ATTENTION, NODE_ALL_REDUCE, NODE_RMSNORM, NODE_ROPE, NODE_EMBEDDING, NODE_SWIGLU, NODE_GELU,
 NODE_ADD, NODE_ARGMAX, NODE_AR_NORM, NODE_ROPE_APPEND, NODE_ATTN_DECODE, NODE_ADVANCE) = range(14)
T_SYMMETRIC = 1


class Graph:
    def __init__(self, ctx: Context):
        self.ctx = ctx
        h = C.c_void_p()
        ctx._check(_lib.hb_graph_create(ctx._h, C.byref(h)))
        self._h = h
        self.meta = {}          # id -> (dtype, shape, stride)

    def close(self):
        if self._h:
            _lib.hb_graph_destroy(self._h)
            self._h = None

    # -- tensors ------------------------------------------------------------------
    def input(self, t: Tensor) -> int:
        i = C.c_int32()
        ct = t.c()
        self.ctx._check(_lib.hb_graph_input(self._h, C.byref(ct), C.byref(i)))
        self.meta[i.value] = (t.dtype, tuple(t.shape), tuple(t.stride))
        return i.value

    def temp(self, shape: Sequence[int], dtype: int = _capi.HB_BF16, symmetric: bool = False) -> int:
        i = C.c_int32()
        arr = (C.c_int64 * len(shape))(*shape)
        self.ctx._check(_lib.hb_graph_temp(self._h, dtype, len(shape), arr, T_SYMMETRIC if symmetric else 0, C.byref(i)))
        self.meta[i.value] = (dtype, tuple(shape), _contig(tuple(shape)))
        return i.value

    def view(self, base: int, offset: int, shape: Sequence[int], stride: Sequence[int]) -> int:
        i = C.c_int32()
        self.ctx._check(_lib.hb_graph_view(self._h, base, offset, len(shape), (C.c_int64 * len(shape))(*shape),
                                           (C.c_int64 * len(stride))(*stride), C.byref(i)))
        self.meta[i.value] = (self.meta[base][0], tuple(shape), tuple(stride))
        return i.value

    # -- nodes --------------------------------------------------------------------
    def _add(self, kind, ins, out, iparam=(), fparam=(), stream=0):
        n = _capi.hb_node()
        n.kind = kind
        n.stream = stream
        for k in range(4):
            n.inputs[k] = ins[k] if k < len(ins) and ins[k] is not None else -1
            n.iparam[k] = iparam[k] if k < len(iparam) else 0
        n.out = out
        for k in range(2):
            n.fparam[k] = fparam[k] if k < len(fparam) else 0.0
        self.ctx._check(_lib.hb_graph_add(self._h, C.byref(n)))
        return out

    def matmul(self, a, b, out, epilogue=_capi.HB_EPI_NONE, residual=None, config_id=-1, gathered=False, weights=False):
        """gathered=True: `a` is the output of the all_reduce_norm node added just before; the
        product waits for its rows block by block instead of for the end of the collective.
        weights=True: `b` is a weight matrix that no node of the graph writes."""
        return self._add(NODE_MATMUL, [a, b, residual], out,
                         [epilogue | (_capi.HB_MATMUL_WEIGHTS_B if weights else 0), config_id, int(gathered)])

    def attention(self, q, k, v, out, causal=True, scale=None, lse=None):
        if scale is None:
            scale = float(self.meta[q][1][-1]) ** -0.5
        return self._add(NODE_ATTENTION, [q, k, v, lse], out, [int(causal)], [scale])

    def all_reduce(self, x, algo=_capi.HB_AR_AUTO, stream=0):
        """stream=1 puts the collective on the context's side stream so that it overlaps
        the nodes that do not depend on it."""
        return self._add(NODE_ALL_REDUCE, [], x, [algo], stream=stream)

    def all_reduce_norm(self, partial, gain, residual_in, residual_out, out, eps=1e-5, gather_only=False,
                        algo=_capi.HB_AR_AUTO, stream=0, ready_words=False):
        """Fused reduce-scatter + residual add + RMSNorm + all-gather (gather_only: publish the
        updated residual rows instead of their norm).  stream=1: on the side stream.
        ready_words: publish a word per block of gathered rows for a ``matmul(..., gathered=True)``."""
        return self._add(NODE_AR_NORM, [partial, gain, residual_in, residual_out], out,
                         [int(gather_only) | (2 if ready_words else 0), algo], [eps], stream=stream)

    def rmsnorm(self, x, gain, out, residual=None, eps=1e-5):
        return self._add(NODE_RMSNORM, [x, gain, residual], out, [], [eps])

    def rope(self, x, seq, heads, head_dim, base=10000.0, pos0=0):
        return self._add(NODE_ROPE, [], x, [seq, heads, head_dim, pos0], [base])

    def rope_append(self, qkv, pos, kv_cache, n_q_heads, n_kv_heads, base=10000.0):
        """RoPE of the new token's q and k heads at pos[0] (in place) and append of k, v to the cache."""
        return self._add(NODE_ROPE_APPEND, [qkv, pos], kv_cache, [n_q_heads, n_kv_heads], [base])

    def attention_decode(self, qkv, kv_cache, pos, out, n_q_heads, n_kv_heads, scale=None, len_hint=0):
        if scale is None:
            scale = float(self.meta[kv_cache][1][-1]) ** -0.5
        return self._add(NODE_ATTN_DECODE, [qkv, kv_cache, pos], out, [n_q_heads, n_kv_heads, len_hint], [scale])

    def advance(self, pos, n=1):
        return self._add(NODE_ADVANCE, [], pos, [n])

    def embedding(self, table, ids, out):
        return self._add(NODE_EMBEDDING, [table, ids], out)

    def swiglu(self, x, out):
        return self._add(NODE_SWIGLU, [x], out)

    def gelu(self, x, out):
        return self._add(NODE_GELU, [x], out)

    def add(self, a, b, out):
        return self._add(NODE_ADD, [a, b], out)

    def argmax(self, x, out):
        return self._add(NODE_ARGMAX, [x], out)

    # -- plan / run -----------------------------------------------------------------
    def plan(self):
        a, s = C.c_size_t(), C.c_size_t()
        self.ctx._check(_lib.hb_graph_plan(self._h, C.byref(a), C.byref(s)))
        return a.value, s.value

    def run(self):
        self.ctx._check(_lib.hb_graph_run(self._h))

    def capture(self):
        """Record one run of the planned graph into a CUDA graph (after one eager run)."""
        self.ctx._check(_lib.hb_graph_capture(self._h))

    def replay(self):
        """Enqueue the captured step with a single call."""
        self.ctx._check(_lib.hb_graph_replay(self._h))

    def run_timed(self, n_nodes: int):
        """One run with per-node device timing; returns a list of milliseconds."""
        ms = (C.c_float * n_nodes)()
        self.ctx._check(_lib.hb_graph_run_timed(self._h, ms, n_nodes))
        return list(ms)

    def describe(self) -> str:
        buf = C.create_string_buffer(1 << 16)
        self.ctx._check(_lib.hb_graph_describe(self._h, buf, len(buf)))
        return buf.value.decode()

    def tensor(self, i: int) -> Tensor:
        p = C.c_void_p()
        self.ctx._check(_lib.hb_graph_tensor_ptr(self._h, i, C.byref(p)))
        dtype, shape, stride = self.meta[i]
        return Tensor(p.value, dtype, shape, stride)


def plan_arena(sizes: Sequence[int], first: Sequence[int], last: Sequence[int]):
    """The executor's placement rule on its own (``hb_plan_arena``; host arithmetic, needs no
    GPU): returns (offsets, total_bytes) for buffers of ``sizes[i]`` bytes alive over node
    indices ``[first[i], last[i]]``."""
    n = len(sizes)
    if not (len(first) == len(last) == n):
        raise ValueError("sizes, first and last must have the same length")
    b = (C.c_size_t * n)(*sizes)
    f = (C.c_int32 * n)(*first)
    l = (C.c_int32 * n)(*last)
    offs = (C.c_size_t * n)()
    total = C.c_size_t(0)
    st = _lib.hb_plan_arena(n, b, f, l, offs, C.byref(total))
    if st != 0:
        raise ValueError(f"hb_plan_arena: status {st}")
    return list(offs), total.value
