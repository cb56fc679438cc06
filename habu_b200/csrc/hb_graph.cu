// Model-IR executor: an ordered list of operator nodes over tensor ids, a memory planner
// that packs planner-owned tensors into one arena by lifetime, and a launcher that walks
// the list and enqueues every node on the context's stream (no host synchronisation
// between nodes).
//
// The shape follows the one piece of the reference that walks a program: a list of
// variant-tagged definitions visited in order and dispatched on the tag
// (`lift_defs_exn`, tree.ml:786-811), with errors returned as values.
//
// Planner: a tensor lives from the first node that writes it to the last node that reads
// it (a view extends its base).  Tensors are placed largest first at the lowest
// 256-byte-aligned offset that does not collide, in time and space, with one already
// placed.  Tensors flagged HB_T_SYMMETRIC (allreduce operands) go to the peer-mapped
// buffer when the context has one that is large enough, so the collective runs over
// NVLink without a staging copy.
#include <stdio.h>
#include <string.h>

#include <algorithm>

#include "hb_internal.h"

struct hb_graph_tensor {
  int kind;                // 0 external, 1 planner-owned, 2 view
  int dtype, rank;
  int64_t shape[4], stride[4];
  void* ptr = nullptr;     // resolved at plan time for kinds 1 and 2
  int base = -1;           // view: tensor viewed
  int64_t offset = 0;      // view: element offset into base
  int flags = 0;
  size_t bytes = 0;
  int first = -1, last = -1;   // lifetime in node indices (owner tensors)
  size_t arena_off = 0;
  bool in_symmetric = false;
};

struct hb_graph {
  hb_ctx* ctx;
  std::vector<hb_graph_tensor> tensors;
  std::vector<hb_node> nodes;
  // two-stream execution: nodes with stream == 1 run on the context's side stream
  std::vector<int> wait_for;            // per node: index of the node on the other stream to wait for, or -1
  std::vector<char> needs_event;        // per node: some node on the other stream waits for it
  std::vector<cudaEvent_t> events;      // per node (created lazily for needs_event nodes)
  cudaEvent_t fork_event = nullptr;
  int last_side_node = -1;
  void* arena = nullptr;
  size_t arena_bytes = 0, symmetric_bytes = 0;
  bool planned = false;
  // replay: the planned node list captured once into a CUDA graph
  bool ran_once = false;                // scratch buffers have their final size
  cudaGraph_t captured = nullptr;
  cudaGraphExec_t exec = nullptr;
  int64_t launches_per_run = 0;
};

namespace {

const char* kNodeNames[] = {"matmul", "attention", "all_reduce", "rmsnorm", "rope", "embedding",
                            "swiglu", "gelu", "add", "argmax", "all_reduce_norm", "rope_append", "attention_decode",
                            "advance"};
size_t elem_size(int dtype) { return dtype == HB_BF16 ? 2 : 4; }

int root_of(const hb_graph* g, int id) {
  while (g->tensors[id].kind == 2) id = g->tensors[id].base;
  return id;
}

bool valid_id(const hb_graph* g, int id) { return id >= 0 && id < (int)g->tensors.size(); }

hb_tensor as_tensor(const hb_graph_tensor& t) {
  hb_tensor o;
  memset(&o, 0, sizeof(o));
  o.ptr = t.ptr;
  o.dtype = t.dtype;
  o.rank = t.rank;
  for (int i = 0; i < t.rank; ++i) { o.shape[i] = t.shape[i]; o.stride[i] = t.stride[i]; }
  return o;
}

int64_t numel(const hb_graph_tensor& t) {
  int64_t n = 1;
  for (int i = 0; i < t.rank; ++i) n *= t.shape[i];
  return n;
}

bool is_contiguous(const hb_graph_tensor& t) {
  int64_t acc = 1;
  for (int i = t.rank - 1; i >= 0; --i) {
    if (t.shape[i] != 1 && t.stride[i] != acc) return false;
    acc *= t.shape[i];
  }
  return true;
}

}  // namespace

extern "C" hb_status hb_graph_create(hb_ctx* ctx, hb_graph** out) {
  if (!ctx || !out) return HB_ERR_INVALID;
  hb_graph* g = new hb_graph();
  g->ctx = ctx;
  *out = g;
  return HB_OK;
}

extern "C" hb_status hb_graph_destroy(hb_graph* g) {
  if (!g) return HB_ERR_INVALID;
  cudaSetDevice(g->ctx->device);
  cudaStreamSynchronize(g->ctx->stream);
  if (g->ctx->side_stream) cudaStreamSynchronize(g->ctx->side_stream);
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->captured) cudaGraphDestroy(g->captured);
  if (g->arena) cudaFree(g->arena);
  for (cudaEvent_t e : g->events)
    if (e) cudaEventDestroy(e);
  if (g->fork_event) cudaEventDestroy(g->fork_event);
  delete g;
  return HB_OK;
}

extern "C" hb_status hb_graph_input(hb_graph* g, const hb_tensor* t, int32_t* id) {
  if (!g || !id) return HB_ERR_INVALID;
  if (!t || !t->ptr) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: external tensor without data");
  if (t->rank < 1 || t->rank > 4) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: rank must be 1..4");
  hb_graph_tensor x;
  x.kind = 0;
  x.dtype = t->dtype;
  x.rank = t->rank;
  for (int i = 0; i < 4; ++i) { x.shape[i] = i < t->rank ? t->shape[i] : 1; x.stride[i] = i < t->rank ? t->stride[i] : 0; }
  x.ptr = t->ptr;
  g->tensors.push_back(x);
  *id = (int32_t)g->tensors.size() - 1;
  g->planned = false;
  return HB_OK;
}

extern "C" hb_status hb_graph_temp(hb_graph* g, int32_t dtype, int32_t rank, const int64_t* shape, int32_t flags,
                                   int32_t* id) {
  if (!g || !id || !shape) return HB_ERR_INVALID;
  if (rank < 1 || rank > 4) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: rank must be 1..4");
  if (dtype != HB_BF16 && dtype != HB_F32 && dtype != HB_I32) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: dtype %d", dtype);
  hb_graph_tensor x;
  x.kind = 1;
  x.dtype = dtype;
  x.rank = rank;
  int64_t acc = 1;
  for (int i = 0; i < 4; ++i) { x.shape[i] = 1; x.stride[i] = 0; }
  for (int i = rank - 1; i >= 0; --i) {
    if (shape[i] <= 0) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: empty dimension");
    x.shape[i] = shape[i];
    x.stride[i] = acc;
    acc *= shape[i];
  }
  x.bytes = (size_t)acc * elem_size(dtype);
  x.flags = flags;
  g->tensors.push_back(x);
  *id = (int32_t)g->tensors.size() - 1;
  g->planned = false;
  return HB_OK;
}

extern "C" hb_status hb_graph_view(hb_graph* g, int32_t base, int64_t offset, int32_t rank, const int64_t* shape,
                                   const int64_t* stride, int32_t* id) {
  if (!g || !id || !shape || !stride) return HB_ERR_INVALID;
  if (!valid_id(g, base)) return hb_fail(g->ctx, HB_ERR_NOT_FOUND, "graph: view of unknown tensor %d", base);
  if (rank < 1 || rank > 4 || offset < 0) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: bad view");
  const hb_graph_tensor& b = g->tensors[base];
  hb_graph_tensor x;
  x.kind = 2;
  x.dtype = b.dtype;
  x.rank = rank;
  int64_t extent = offset;
  for (int i = 0; i < 4; ++i) { x.shape[i] = 1; x.stride[i] = 0; }
  for (int i = 0; i < rank; ++i) {
    if (shape[i] <= 0 || stride[i] < 0) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: bad view dimension");
    x.shape[i] = shape[i];
    x.stride[i] = stride[i];
    extent += (shape[i] - 1) * stride[i];
  }
  // bounds: a view of a planner-owned tensor must stay inside it (the extent of caller-owned
  // memory is not known here)
  {
    int64_t abs_extent = extent;
    int id = base;
    while (g->tensors[id].kind == 2) { abs_extent += g->tensors[id].offset; id = g->tensors[id].base; }
    if (g->tensors[id].kind == 1 && abs_extent >= numel(g->tensors[id]))
      return hb_fail(g->ctx, HB_ERR_INVALID, "graph: view reaches past the end of tensor %d", base);
  }
  x.base = base;
  x.offset = offset;
  g->tensors.push_back(x);
  *id = (int32_t)g->tensors.size() - 1;
  g->planned = false;
  return HB_OK;
}

extern "C" hb_status hb_graph_add(hb_graph* g, const hb_node* n) {
  if (!g || !n) return HB_ERR_INVALID;
  if (n->kind < 0 || n->kind > HB_NODE_ADVANCE) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: unknown node kind %d", n->kind);
  static const int n_in[] = {2, 3, 0, 2, 0, 2, 1, 1, 2, 1, 1, 2, 3, 0};   // required leading inputs per kind
  for (int i = 0; i < 4; ++i) {
    if (i < n_in[n->kind] && !valid_id(g, n->in[i]))
      return hb_fail(g->ctx, HB_ERR_NOT_FOUND, "graph: %s node input %d names unknown tensor %d", kNodeNames[n->kind], i, n->in[i]);
    if (i >= n_in[n->kind] && n->in[i] != -1 && !valid_id(g, n->in[i]))
      return hb_fail(g->ctx, HB_ERR_NOT_FOUND, "graph: %s node optional input %d names unknown tensor %d", kNodeNames[n->kind], i, n->in[i]);
  }
  if (!valid_id(g, n->out)) return hb_fail(g->ctx, HB_ERR_NOT_FOUND, "graph: %s node output names unknown tensor %d", kNodeNames[n->kind], n->out);
  // Only the collective nodes may run on the side stream.  The executor orders nodes on
  // different streams by the byte ranges of their tensors; compute nodes also share state it
  // cannot see (the stream-K workspace and tickets, the RoPE angle table, the attention work
  // counters), so two of them on different streams could race on it.
  if (n->stream != 0 && n->stream != 1) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: stream must be 0 or 1");
  if (n->stream == 1 && n->kind != HB_NODE_ALL_REDUCE && n->kind != HB_NODE_AR_NORM)
    return hb_fail(g->ctx, HB_ERR_UNSUPPORTED, "graph: only all_reduce and all_reduce_norm nodes may run on the side stream (%s node)",
                   kNodeNames[n->kind]);
  g->nodes.push_back(*n);
  g->planned = false;
  return HB_OK;
}

// Arena placement by lifetime: buffers are taken largest first (ties by index) and each goes to
// the lowest 256-byte-aligned offset that is free during its whole lifetime [first, last]
// (node indices, inclusive).  Pure host arithmetic; the executor calls it once per arena.
extern "C" hb_status hb_plan_arena(int32_t n, const size_t* bytes, const int32_t* first, const int32_t* last,
                                   size_t* offsets, size_t* total) {
  if (n < 0 || !total || (n > 0 && (!bytes || !first || !last || !offsets))) return HB_ERR_INVALID;
  for (int i = 0; i < n; ++i)
    if (first[i] < 0 || last[i] < first[i]) return HB_ERR_INVALID;
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  std::vector<int> order(n);
  for (int i = 0; i < n; ++i) order[i] = i;
  std::sort(order.begin(), order.end(), [&](int a, int b) {
    if (bytes[a] != bytes[b]) return bytes[a] > bytes[b];
    return a < b;
  });
  std::vector<int> placed;
  size_t top = 0;
  for (int id : order) {
    const size_t sz = up(bytes[id]);
    std::vector<std::pair<size_t, size_t>> busy;   // [begin, end) of the buffers alive at the same time
    for (int o : placed) {
      if (last[o] < first[id] || last[id] < first[o]) continue;
      busy.emplace_back(offsets[o], offsets[o] + up(bytes[o]));
    }
    std::sort(busy.begin(), busy.end());
    size_t off = 0;
    for (const auto& b : busy) {
      if (off + sz <= b.first) break;
      if (b.second > off) off = b.second;
    }
    offsets[id] = off;
    placed.push_back(id);
    if (off + sz > top) top = off + sz;
  }
  *total = top;
  return HB_OK;
}

extern "C" hb_status hb_graph_plan(hb_graph* g, size_t* arena_bytes, size_t* symmetric_bytes) {
  if (!g) return HB_ERR_INVALID;
  hb_ctx* ctx = g->ctx;
  // ---- lifetimes
  for (auto& t : g->tensors) { t.first = -1; t.last = -1; }
  auto touch = [&](int id, int node) {
    if (id < 0) return;
    hb_graph_tensor& r = g->tensors[root_of(g, id)];
    if (r.first < 0) r.first = node;
    r.last = node;
  };
  for (int i = 0; i < (int)g->nodes.size(); ++i) {
    for (int k = 0; k < 4; ++k) touch(g->nodes[i].in[k], i);
    touch(g->nodes[i].out, i);
  }
  // a planner-owned tensor that is read before any node wrote it would read garbage
  for (int i = 0; i < (int)g->nodes.size(); ++i) {
    const hb_node& n = g->nodes[i];
    for (int k = 0; k < 4; ++k) {
      if (n.in[k] < 0) continue;
      if (n.kind == HB_NODE_AR_NORM && k == 3) continue;   // residual_out is written, not read
      const int r = root_of(g, n.in[k]);
      if (g->tensors[r].kind != 1) continue;
      bool written = false;
      for (int j = 0; j < i && !written; ++j)
        written = root_of(g, g->nodes[j].out) == r ||
                  (g->nodes[j].kind == HB_NODE_AR_NORM && g->nodes[j].in[3] >= 0 && root_of(g, g->nodes[j].in[3]) == r);
      if (!written)
        return hb_fail(ctx, HB_ERR_INVALID, "graph: node %d (%s) reads planner-owned tensor %d before any node writes it", i,
                       kNodeNames[n.kind], n.in[k]);
    }
  }
  // ---- placement, one pass per arena (0 ordinary, 1 symmetric)
  const bool have_sym = ctx->p2p.local != nullptr;
  size_t totals[2] = {0, 0};
  for (int pass = 0; pass < 2; ++pass) {
    std::vector<int> ids;
    for (int i = 0; i < (int)g->tensors.size(); ++i) {
      hb_graph_tensor& t = g->tensors[i];
      if (t.kind != 1 || t.first < 0) continue;
      const bool sym = (t.flags & HB_T_SYMMETRIC) != 0;
      if ((int)sym == pass) ids.push_back(i);
    }
    std::vector<size_t> bytes(ids.size()), offs(ids.size());
    std::vector<int32_t> first(ids.size()), last(ids.size());
    for (size_t k = 0; k < ids.size(); ++k) {
      bytes[k] = g->tensors[ids[k]].bytes;
      first[k] = g->tensors[ids[k]].first;
      last[k] = g->tensors[ids[k]].last;
    }
    hb_status st = hb_plan_arena((int32_t)ids.size(), bytes.data(), first.data(), last.data(), offs.data(), &totals[pass]);
    if (st != HB_OK) return hb_fail(ctx, st, "graph: arena planning failed");
    for (size_t k = 0; k < ids.size(); ++k) {
      g->tensors[ids[k]].arena_off = offs[k];
      g->tensors[ids[k]].in_symmetric = pass == 1;
    }
  }
  // symmetric tensors fall back to the ordinary arena when no peer buffer can hold them
  const bool sym_fits = have_sym && totals[1] <= ctx->p2p.bytes;
  size_t sym_base_in_arena = 0;
  size_t need = totals[0];
  if (!sym_fits && totals[1] > 0) {
    sym_base_in_arena = (totals[0] + 255) & ~size_t(255);
    need = sym_base_in_arena + totals[1];
  }
  if (need > g->arena_bytes) {
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaSetDevice");
    if (g->arena) { cudaStreamSynchronize(ctx->stream); cudaFree(g->arena); g->arena = nullptr; g->arena_bytes = 0; }
    e = cudaMalloc(&g->arena, need);
    if (e != cudaSuccess) { cudaGetLastError(); return hb_fail(ctx, HB_ERR_NOMEM, "graph: cannot allocate a %zu-byte arena", need); }
    g->arena_bytes = need;
  }
  for (auto& t : g->tensors) {
    if (t.kind != 1 || t.first < 0) continue;
    if (t.in_symmetric && sym_fits) t.ptr = static_cast<char*>(ctx->p2p.local) + t.arena_off;
    else if (t.in_symmetric) { t.ptr = static_cast<char*>(g->arena) + sym_base_in_arena + t.arena_off; }
    else t.ptr = static_cast<char*>(g->arena) + t.arena_off;
  }
  for (auto& t : g->tensors) {
    if (t.kind != 2) continue;
    // resolve view chains: pointer = root pointer + accumulated element offsets
    int64_t off = 0;
    int id = (int)(&t - &g->tensors[0]);
    while (g->tensors[id].kind == 2) { off += g->tensors[id].offset; id = g->tensors[id].base; }
    const hb_graph_tensor& r = g->tensors[id];
    t.ptr = r.ptr ? static_cast<char*>(r.ptr) + off * (int64_t)elem_size(r.dtype) : nullptr;
  }
  g->symmetric_bytes = totals[1];
  // ---- cross-stream dependencies, on byte ranges (planner-owned tensors may share memory)
  {
    const int nn = (int)g->nodes.size();
    struct Range { const char* lo; const char* hi; bool write; };
    auto range_of = [&](int id, bool write) {
      const hb_graph_tensor& t = g->tensors[id];
      int64_t ext = 1;
      for (int i = 0; i < t.rank; ++i) ext += (t.shape[i] - 1) * t.stride[i];
      const char* lo = static_cast<const char*>(t.ptr);
      return Range{lo, lo + ext * (int64_t)elem_size(t.dtype), write};
    };
    std::vector<std::vector<Range>> foot(nn);
    bool any_side = false;
    for (int i = 0; i < nn; ++i) {
      const hb_node& n = g->nodes[i];
      if (n.stream != 0) any_side = true;
      for (int k = 0; k < 4; ++k)
        if (n.in[k] >= 0)
          foot[i].push_back(range_of(n.in[k], (n.kind == HB_NODE_RMSNORM && k == 2) || (n.kind == HB_NODE_AR_NORM && k == 3) ||
                                                  (n.kind == HB_NODE_ATTENTION && k == 3) || (n.kind == HB_NODE_ROPE_APPEND && k == 0)));   // inputs the node writes
      foot[i].push_back(range_of(n.out, true));
    }
    g->wait_for.assign(nn, -1);
    g->needs_event.assign(nn, 0);
    g->last_side_node = -1;
    if (any_side) {
      if (!ctx->side_stream) {
        // highest priority: when SM resources free up, the collective's CTAs are placed before
        // the queued compute kernels', so it starts as soon as its producer finishes
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        cudaError_t e = cudaStreamCreateWithPriority(&ctx->side_stream, cudaStreamNonBlocking, hi);
        if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaStreamCreate(side)");
      }
      for (int i = 0; i < nn; ++i) {
        if (g->nodes[i].stream != 0) g->last_side_node = i;
        for (int j = i - 1; j >= 0; --j) {
          if ((g->nodes[j].stream != 0) == (g->nodes[i].stream != 0)) continue;
          bool conflict = false;
          // a gathered matmul is ordered behind the collective that writes its A by the "rows
          // ready" words, not by an event: that one pair of ranges is no conflict
          const bool by_words = g->nodes[i].kind == HB_NODE_MATMUL && g->nodes[i].iparam[2] != 0 &&
                                g->nodes[j].kind == HB_NODE_AR_NORM;
          for (size_t ai = 0; ai < foot[i].size(); ++ai)
            for (size_t bi = 0; bi < foot[j].size(); ++bi) {
              const Range& a = foot[i][ai];
              const Range& b = foot[j][bi];
              if (by_words && ai == 0 && bi + 1 == foot[j].size()) continue;
              if ((a.write || b.write) && a.lo < b.hi && b.lo < a.hi) conflict = true;
            }
          if (conflict) { g->wait_for[i] = j; g->needs_event[j] = 1; break; }   // the latest one covers earlier ones
        }
      }
      if (g->last_side_node >= 0) g->needs_event[g->last_side_node] = 1;
      g->events.resize(nn, nullptr);
      for (int i = 0; i < nn; ++i)
        if (g->needs_event[i] && !g->events[i] &&
            cudaEventCreateWithFlags(&g->events[i], cudaEventDisableTiming) != cudaSuccess)
          return hb_fail(ctx, HB_ERR_CUDA, "graph: cannot create events");
      if (!g->fork_event && cudaEventCreateWithFlags(&g->fork_event, cudaEventDisableTiming) != cudaSuccess)
        return hb_fail(ctx, HB_ERR_CUDA, "graph: cannot create events");
    }
  }
  g->planned = true;
  g->ran_once = false;                  // addresses may have moved: a captured replay is stale
  if (g->exec) { cudaGraphExecDestroy(g->exec); g->exec = nullptr; }
  if (g->captured) { cudaGraphDestroy(g->captured); g->captured = nullptr; }
  if (arena_bytes) *arena_bytes = need;
  if (symmetric_bytes) *symmetric_bytes = totals[1];
  return HB_OK;
}

static hb_status run_node(hb_graph* g, int i) {
  hb_ctx* ctx = g->ctx;
  {
    const hb_node& n = g->nodes[i];
    auto T = [&](int id) -> const hb_graph_tensor& { return g->tensors[id]; };
    hb_status st = HB_OK;
    switch (n.kind) {
      case HB_NODE_MATMUL: {
        hb_tensor a = as_tensor(T(n.in[0])), b = as_tensor(T(n.in[1])), c = as_tensor(T(n.out));
        hb_matmul_opts o = {n.iparam[0], n.iparam[1], nullptr, 0};
        if ((n.iparam[0] & 0xff) == HB_EPI_RESIDUAL) {
          if (n.in[2] < 0) { st = hb_fail(ctx, HB_ERR_INVALID, "graph: residual epilogue without a residual tensor"); break; }
          o.residual = T(n.in[2]).ptr;
          o.residual_ld = T(n.in[2]).stride[0];
        }
        st = n.iparam[2] ? hb_matmul_gathered(ctx, &a, &b, &c, &o) : hb_matmul(ctx, &a, &b, &c, &o);
        break;
      }
      case HB_NODE_ATTENTION: {
        hb_tensor q = as_tensor(T(n.in[0])), k = as_tensor(T(n.in[1])), v = as_tensor(T(n.in[2])), o = as_tensor(T(n.out));
        hb_attn_opts opts = {n.iparam[0], n.fparam[0], n.in[3] >= 0 ? T(n.in[3]).ptr : nullptr, -1};
        st = hb_attention(ctx, &q, &k, &v, &o, &opts);
        break;
      }
      case HB_NODE_ALL_REDUCE: {
        const hb_graph_tensor& x = T(n.out);
        if (!is_contiguous(x)) { st = hb_fail(ctx, HB_ERR_UNSUPPORTED, "graph: all_reduce needs a contiguous tensor"); break; }
        st = hb_all_reduce(ctx, x.ptr, numel(x), x.dtype, n.iparam[0]);
        break;
      }
      case HB_NODE_RMSNORM: {
        const hb_graph_tensor& x = T(n.in[0]);
        if (x.rank != 2 || !is_contiguous(x) || !is_contiguous(T(n.out))) { st = hb_fail(ctx, HB_ERR_UNSUPPORTED, "graph: rmsnorm needs contiguous [rows, cols]"); break; }
        st = hb_rmsnorm(ctx, x.ptr, T(n.in[1]).ptr, T(n.out).ptr, n.in[2] >= 0 ? T(n.in[2]).ptr : nullptr, x.shape[0], x.shape[1],
                        n.fparam[0]);
        break;
      }
      case HB_NODE_ROPE: {
        const hb_graph_tensor& x = T(n.out);   // [tokens, heads * head_dim] with a row stride
        if (x.rank != 2 || x.stride[1] != 1) { st = hb_fail(ctx, HB_ERR_UNSUPPORTED, "graph: rope needs [tokens, heads*head_dim] rows"); break; }
        st = hb_rope(ctx, x.ptr, x.shape[0], n.iparam[0], n.iparam[1], n.iparam[2], x.stride[0], n.fparam[0], n.iparam[3]);
        break;
      }
      case HB_NODE_EMBEDDING: {
        const hb_graph_tensor& tab = T(n.in[0]);
        st = hb_embedding(ctx, tab.ptr, static_cast<const int32_t*>(T(n.in[1]).ptr), T(n.out).ptr, T(n.in[1]).shape[0],
                          tab.shape[0], tab.shape[1]);
        break;
      }
      case HB_NODE_SWIGLU: {
        const hb_graph_tensor& x = T(n.in[0]);
        st = hb_swiglu(ctx, x.ptr, T(n.out).ptr, x.shape[0], x.shape[1] / 2);
        break;
      }
      case HB_NODE_GELU:
        st = hb_gelu(ctx, T(n.in[0]).ptr, T(n.out).ptr, numel(T(n.in[0])));
        break;
      case HB_NODE_ADD:
        st = hb_add(ctx, T(n.in[0]).ptr, T(n.in[1]).ptr, T(n.out).ptr, numel(T(n.in[0])));
        break;
      case HB_NODE_AR_NORM: {
        const hb_graph_tensor& x = T(n.in[0]);
        if (x.rank != 2 || !is_contiguous(x) || !is_contiguous(T(n.out)) || n.in[2] < 0 || n.in[3] < 0) {
          st = hb_fail(ctx, HB_ERR_INVALID, "graph: all_reduce_norm needs contiguous [rows, cols], a residual input and a residual output");
          break;
        }
        st = hb_all_reduce_norm(ctx, x.ptr, n.in[1] >= 0 ? T(n.in[1]).ptr : nullptr, T(n.in[2]).ptr, T(n.in[3]).ptr, T(n.out).ptr,
                                x.shape[0], x.shape[1], n.fparam[0], n.iparam[0], n.iparam[1]);
        break;
      }
      case HB_NODE_ROPE_APPEND: {
        const hb_graph_tensor& x = T(n.in[0]);     // [batch, row] new-token projections
        const hb_graph_tensor& kv = T(n.out);      // [2*batch, s_max, kv_heads, 128]
        if (x.rank != 2 || x.stride[1] != 1 || kv.rank != 4 || !is_contiguous(kv) || kv.shape[0] != 2 * x.shape[0] ||
            kv.shape[2] != n.iparam[1] || T(n.in[1]).dtype != HB_I32) {
          st = hb_fail(ctx, HB_ERR_INVALID, "graph: rope_append needs qkv [batch, row], an i32 position and a contiguous cache [2*batch, s_max, kv_heads, 128]");
          break;
        }
        st = hb_rope_append(ctx, x.ptr, x.stride[0], kv.ptr, static_cast<const int32_t*>(T(n.in[1]).ptr), x.shape[0], n.iparam[0],
                            n.iparam[1], kv.shape[3], kv.shape[1], n.fparam[0]);
        break;
      }
      case HB_NODE_ATTN_DECODE: {
        const hb_graph_tensor& x = T(n.in[0]);
        const hb_graph_tensor& kv = T(n.in[1]);
        const hb_graph_tensor& o = T(n.out);
        if (x.rank != 2 || x.stride[1] != 1 || kv.rank != 4 || !is_contiguous(kv) || kv.shape[0] != 2 * x.shape[0] ||
            kv.shape[2] != n.iparam[1] || T(n.in[2]).dtype != HB_I32 || !is_contiguous(o) ||
            numel(o) != x.shape[0] * n.iparam[0] * kv.shape[3]) {
          st = hb_fail(ctx, HB_ERR_INVALID, "graph: attention_decode needs qkv [batch, row], a contiguous cache, an i32 position and a contiguous [batch, q_heads*128] output");
          break;
        }
        st = hb_attention_decode(ctx, x.ptr, x.stride[0], kv.ptr, static_cast<const int32_t*>(T(n.in[2]).ptr), o.ptr, x.shape[0],
                                 n.iparam[0], n.iparam[1], kv.shape[3], kv.shape[1], n.iparam[2], n.fparam[0]);
        break;
      }
      case HB_NODE_ADVANCE:
        if (T(n.out).dtype != HB_I32) { st = hb_fail(ctx, HB_ERR_INVALID, "graph: advance needs an i32 position"); break; }
        st = hb_advance_pos(ctx, static_cast<int32_t*>(T(n.out).ptr), n.iparam[0]);
        break;
      case HB_NODE_ARGMAX: {
        const hb_graph_tensor& x = T(n.in[0]);
        st = hb_argmax(ctx, x.ptr, static_cast<int32_t*>(T(n.out).ptr), x.shape[0], x.shape[1]);
        break;
      }
      default:
        st = hb_fail(ctx, HB_ERR_INVALID, "graph: unknown node kind %d", n.kind);
    }
    if (st != HB_OK) {
      std::string inner = ctx->err;
      return hb_fail(ctx, st, "graph node %d (%s): %s", i, kNodeNames[n.kind], inner.c_str());
    }
  }
  return HB_OK;
}

extern "C" hb_status hb_graph_run(hb_graph* g) {
  if (!g) return HB_ERR_INVALID;
  if (!g->planned) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: call hb_graph_plan before hb_graph_run");
  hb_ctx* ctx = g->ctx;
  cudaStream_t main_stream = ctx->stream;
  const bool two = g->last_side_node >= 0;
  if (two) {   // the side stream starts after everything already queued on the main stream
    cudaEventRecord(g->fork_event, main_stream);
    cudaStreamWaitEvent(ctx->side_stream, g->fork_event, 0);
  }
  hb_status st = HB_OK;
  for (int i = 0; i < (int)g->nodes.size() && st == HB_OK; ++i) {
    cudaStream_t s = (two && g->nodes[i].stream != 0) ? ctx->side_stream : main_stream;
    if (two && g->wait_for[i] >= 0) cudaStreamWaitEvent(s, g->events[g->wait_for[i]], 0);
    ctx->stream = s;
    st = run_node(g, i);
    ctx->stream = main_stream;
    if (two && g->needs_event[i]) cudaEventRecord(g->events[i], s);
  }
  if (two) cudaStreamWaitEvent(main_stream, g->events[g->last_side_node], 0);   // join
  if (st == HB_OK) g->ran_once = true;
  return st;
}

// Replay.  hb_graph_capture records one run of the planned node list -- both streams, with
// the event edges between them -- into a CUDA graph and instantiates it; hb_graph_replay then
// enqueues the whole step with one call, which removes the per-node launch gaps that dominate
// short steps (a decode step is about thirty kernels of a few microseconds each).
//   - The graph must have run once eagerly since it was planned: the context's scratch buffers
//     grow on first use, and growing (free + allocate + synchronise) is not capturable.
//   - Everything a node reads from the host is frozen at capture time: tensor addresses,
//     shapes, configuration choices.  Values that change from step to step must live in device
//     memory (the decode position does).
//   - Graphs with collective nodes are refused: the cross-GPU handshakes count calls on the
//     host, so a replayed launch would reuse a stale count.
//   - The RoPE angle table is rebuilt inside the captured step, so a replay does not depend on
//     what other RoPE calls the context has served in between.
extern "C" hb_status hb_graph_capture(hb_graph* g) {
  if (!g) return HB_ERR_INVALID;
  hb_ctx* ctx = g->ctx;
  if (!g->planned) return hb_fail(ctx, HB_ERR_INVALID, "graph: call hb_graph_plan before hb_graph_capture");
  if (!g->ran_once) return hb_fail(ctx, HB_ERR_INVALID, "graph: run the planned graph once (hb_graph_run) before capturing it");
  for (const hb_node& n : g->nodes)
    if (n.kind == HB_NODE_ALL_REDUCE || n.kind == HB_NODE_AR_NORM)
      if (ctx->world > 1) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "graph: a graph with collective nodes cannot be captured");
  if (g->exec) { cudaGraphExecDestroy(g->exec); g->exec = nullptr; }
  if (g->captured) { cudaGraphDestroy(g->captured); g->captured = nullptr; }
  HB_CUDA(ctx, cudaSetDevice(ctx->device));
  HB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->rope_seq = 0;                                   // the table kernel becomes part of the capture
  const int64_t l0 = ctx->launches;
  cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed);
  if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaStreamBeginCapture");
  hb_status st = hb_graph_run(g);
  std::string inner = ctx->err;
  cudaGraph_t graph = nullptr;
  e = cudaStreamEndCapture(ctx->stream, &graph);
  if (st != HB_OK) {
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    return hb_fail(ctx, st, "graph: capture failed: %s", inner.c_str());
  }
  if (e != cudaSuccess || !graph) { cudaGetLastError(); return hb_fail(ctx, HB_ERR_CUDA, "graph: cudaStreamEndCapture: %s", cudaGetErrorString(e)); }
  e = cudaGraphInstantiate(&g->exec, graph, 0);
  if (e != cudaSuccess) { cudaGraphDestroy(graph); cudaGetLastError(); return hb_fail(ctx, HB_ERR_CUDA, "graph: cudaGraphInstantiate: %s", cudaGetErrorString(e)); }
  g->captured = graph;
  g->launches_per_run = ctx->launches - l0;
  ctx->launches = l0;                                  // nothing ran: the launches were recorded, not executed
  return HB_OK;
}

extern "C" hb_status hb_graph_replay(hb_graph* g) {
  if (!g) return HB_ERR_INVALID;
  if (!g->exec) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: call hb_graph_capture before hb_graph_replay");
  cudaError_t e = cudaGraphLaunch(g->exec, g->ctx->stream);
  if (e != cudaSuccess) return hb_check_cuda(g->ctx, e, "cudaGraphLaunch");
  g->ctx->launches += g->launches_per_run;
  return HB_OK;
}

// Runs the graph once with a CUDA event between nodes and reports each node's device
// time in milliseconds (ms[i] for node i, up to `n` entries).  Synchronises the stream.
extern "C" hb_status hb_graph_run_timed(hb_graph* g, float* ms, int32_t n) {
  if (!g || !ms) return HB_ERR_INVALID;
  hb_ctx* ctx = g->ctx;
  if (!g->planned) return hb_fail(ctx, HB_ERR_INVALID, "graph: call hb_graph_plan before hb_graph_run_timed");
  const int count = (int)g->nodes.size();
  std::vector<cudaEvent_t> ev(count + 1);
  for (auto& e : ev)
    if (cudaEventCreate(&e) != cudaSuccess) return hb_fail(ctx, HB_ERR_CUDA, "graph: cannot create events");
  hb_status st = HB_OK;
  cudaEventRecord(ev[0], ctx->stream);
  for (int i = 0; i < count && st == HB_OK; ++i) {
    st = run_node(g, i);
    cudaEventRecord(ev[i + 1], ctx->stream);
  }
  if (st == HB_OK) st = hb_sync(ctx);
  if (st == HB_OK)
    for (int i = 0; i < count && i < n; ++i) cudaEventElapsedTime(&ms[i], ev[i], ev[i + 1]);
  for (auto& e : ev) cudaEventDestroy(e);
  return st;
}

// Text listing of the planned graph: one line per node, then one per planner-owned
// tensor with its lifetime and arena offset.
extern "C" hb_status hb_graph_describe(hb_graph* g, char* buf, size_t len) {
  if (!g || !buf || len == 0) return HB_ERR_INVALID;
  std::string s;
  char line[256];
  for (int i = 0; i < (int)g->nodes.size(); ++i) {
    const hb_node& n = g->nodes[i];
    snprintf(line, sizeof(line), "n%d %s in(%d,%d,%d,%d) out %d\n", i, kNodeNames[n.kind], n.in[0], n.in[1], n.in[2], n.in[3], n.out);
    s += line;
  }
  for (int i = 0; i < (int)g->tensors.size(); ++i) {
    const hb_graph_tensor& t = g->tensors[i];
    if (t.kind != 1) continue;
    snprintf(line, sizeof(line), "t%d %s bytes %zu live [%d,%d] %s+%zu\n", i, t.dtype == HB_BF16 ? "bf16" : t.dtype == HB_F32 ? "f32" : "i32",
             t.bytes, t.first, t.last, t.in_symmetric ? "sym" : "arena", t.arena_off);
    s += line;
  }
  snprintf(line, sizeof(line), "arena %zu symmetric %zu\n", g->arena_bytes, g->symmetric_bytes);
  s += line;
  if (s.size() + 1 > len) return hb_fail(g->ctx, HB_ERR_NOMEM, "graph: describe needs %zu bytes", s.size() + 1);
  memcpy(buf, s.c_str(), s.size() + 1);
  return HB_OK;
}

extern "C" hb_status hb_graph_tensor_ptr(hb_graph* g, int32_t id, void** ptr) {
  if (!g || !ptr) return HB_ERR_INVALID;
  if (!valid_id(g, id)) return hb_fail(g->ctx, HB_ERR_NOT_FOUND, "graph: unknown tensor %d", id);
  if (!g->planned) return hb_fail(g->ctx, HB_ERR_INVALID, "graph: not planned");
  *ptr = g->tensors[id].ptr;
  return HB_OK;
}
