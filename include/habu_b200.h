/*
 * habu_b200.h -- C ABI of libhabu_b200.so, the sm_100a kernel library behind the
 * model-IR executor's dense hot path (matmul / attention / collective nodes and the
 * autotune entry point).
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an
 * `hb_status`, and never throws, aborts or traps.  All operators are asynchronous on
 * the context's stream; `hb_sync` is the only blocking call, so a foreign runtime
 * (e.g. OCaml `foreign_stubs`) can release its runtime lock there and nowhere else.
 *
 * Reference interface: the reference project (joelreymont/habu) has NO operator, plugin
 * or FFI surface for this path -- `src/lib/dune:1-12` holds only `library`, `ocamllex`
 * and `menhir` stanzas, with no `foreign_stubs` and no `external` declarations anywhere.
 * The conventions the reference does pin are mirrored where they apply:
 *   - errors are values, never exceptions: `` `Invalid | `Duplicate | `Not_found ``
 *     of `src/lib/error.ml:18-26` map to HB_ERR_INVALID / HB_ERR_DUPLICATE /
 *     HB_ERR_NOT_FOUND;
 *   - constructors validate and return a result (`Space.make`, `src/lib/sleigh.ml:50-62`):
 *     every operator validates its descriptors on the host before any launch;
 *   - a list of variant-tagged definitions is walked in order and dispatched on its tag
 *     (`lift_defs_exn`, `tree.ml:786-811`): `hb_graph_*` keeps the same shape.
 */
#ifndef HABU_B200_H
#define HABU_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t hb_status;
enum {
  HB_OK = 0,
  HB_ERR_INVALID = 1,     /* `Invalid   (src/lib/error.ml:19) */
  HB_ERR_NOT_FOUND = 2,   /* `Not_found (src/lib/error.ml:21) */
  HB_ERR_DUPLICATE = 3,   /* `Duplicate (src/lib/error.ml:20) */
  HB_ERR_CUDA = 4,
  HB_ERR_NCCL = 5,
  HB_ERR_TIMEOUT = 6,     /* a bounded device-side wait gave up */
  HB_ERR_UNSUPPORTED = 7,
  HB_ERR_NOMEM = 8
};

enum { HB_F32 = 0, HB_BF16 = 1, HB_I32 = 2 };

/* POD tensor view: `ptr` is a DEVICE pointer, strides are in ELEMENTS. */
typedef struct hb_tensor {
  void* ptr;
  int32_t dtype;
  int32_t rank;
  int64_t shape[4];
  int64_t stride[4];
} hb_tensor;

typedef struct hb_ctx hb_ctx;

/* ---- context / memory (no reference counterpart: the reference never leaves the host) */
hb_status hb_ctx_create(int32_t device, hb_ctx** out);
hb_status hb_ctx_destroy(hb_ctx* ctx);
/* Use a caller-owned CUDA stream (a cudaStream_t passed as void*); NULL restores the
 * context's own stream. */
hb_status hb_ctx_set_stream(hb_ctx* ctx, void* cuda_stream);
const char* hb_last_error_string(hb_ctx* ctx);
hb_status hb_alloc(hb_ctx* ctx, size_t bytes, void** dev_ptr);
hb_status hb_free(hb_ctx* ctx, void* dev_ptr);
hb_status hb_upload(hb_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
hb_status hb_download(hb_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
/* Blocks until the stream drains; returns HB_ERR_TIMEOUT if any kernel's bounded wait
 * gave up since the last call, HB_ERR_CUDA on an asynchronous CUDA error. */
hb_status hb_sync(hb_ctx* ctx);
/* Number of this library's kernels launched through `ctx` since creation. */
int64_t hb_launch_count(hb_ctx* ctx);
int32_t hb_sm_count(hb_ctx* ctx);

/* ---- model-IR matmul node ---------------------------------------------------------
 * C[M,N] = epilogue(A[M,K] . B[K,N]).  bf16 operands, fp32 accumulation in tensor
 * memory, bf16 output (HB_BF16), or fp32 throughout on CUDA cores (HB_F32).
 * Operand layouts are taken from the strides: A is K-contiguous (row-major) or
 * M-contiguous; B is K-contiguous ("column-major B", stride[0] == 1) or N-contiguous.
 * C is row-major.  Replaces: nothing -- the reference has no matmul; `MUL`/`FMUL`
 * (`src/lib/sleigh.ml:219,224`) are syntax constructors that are never evaluated. */
enum {
  HB_EPI_NONE = 0,
  HB_EPI_GELU = 1,          /* erf-exact GELU */
  HB_EPI_SWIGLU = 2,        /* B's N columns interleave (gate,up); C has N/2 columns */
  HB_EPI_RESIDUAL = 3       /* C = A.B + R, R row-major bf16 shaped like C */
};
/* OR-ed into hb_matmul_opts.epilogue: B is a weight matrix -- nothing still in flight on the GPU
 * writes it.  The stream-K kernel (M <= 64) may then start streaming B in while the kernel in
 * front of it on the stream is still running (programmatic dependent launch); A, C and the
 * scratch are touched only after that kernel has finished.  Without the flag the launch keeps
 * plain stream order. */
#define HB_MATMUL_WEIGHTS_B 0x100
typedef struct hb_matmul_opts {
  int32_t epilogue;         /* HB_EPI_*, optionally | HB_MATMUL_WEIGHTS_B */
  int32_t config_id;        /* -1: use the autotune cache / heuristic */
  const void* residual;     /* device pointer, HB_EPI_RESIDUAL only */
  int64_t residual_ld;      /* elements */
} hb_matmul_opts;
hb_status hb_matmul(hb_ctx* ctx, const hb_tensor* A, const hb_tensor* B, hb_tensor* C,
                    const hb_matmul_opts* opts);
/* Same node for an A that is the gathered output of the hb_all_reduce_norm call enqueued just
 * before it: the loader waits block by block for the rows to land ("rows ready" words the
 * collective publishes) and visits this rank's own rows first, so the call may be enqueued on
 * a stream that does not wait for the collective and the product overlaps the all-gather.
 * Needs row-major bf16 A with more than 64 rows; with one rank it is hb_matmul.  No
 * reference counterpart. */
hb_status hb_matmul_gathered(hb_ctx* ctx, const hb_tensor* A, const hb_tensor* B, hb_tensor* C,
                             const hb_matmul_opts* opts);
/* Same node with HOST buffers: uploads A and B, runs, downloads C, synchronises.
 * A is [M,K] row-major, B is column-major (K contiguous per column), C row-major. */
hb_status hb_matmul_host(hb_ctx* ctx, const void* A_host, const void* B_host, void* C_host,
                         int64_t M, int64_t N, int64_t K, int32_t dtype);

/* Skinny matmul (M <= 64) for callers that cannot allocate device memory when they need
 * the product -- a latency-critical serving loop that bans allocator locks and the device
 * synchronisation cudaMalloc/cudaFree may imply, a foreign-runtime callback that must not
 * block in the driver, or a process whose device memory was handed out in full at start-up.
 * This entry point has no counterpart in the reference and needs no hb_ctx: the split-K
 * scratch is a static device array inside the library (about 4 MiB per GPU, held until
 * the process exits).  A [M,K] row-major, B column-major (N rows of K), C [M,N] row-major,
 * all bf16 device pointers; `device` must be the calling thread's current device and
 * `cuda_stream` a cudaStream_t (NULL = default stream).  Asynchronous.
 *   - Limit: ceil(N/128) * segments * 128 * roundup16(M) <= 2^20 partial floats (segments:
 *     the K ranges that can share one column tile, 4 at N=K=8192) and at most 1024 column
 *     tiles; anything larger returns HB_ERR_UNSUPPORTED with a message.
 *   - The first call on a device looks up the static arrays' device addresses and sets
 *     the kernel's shared-memory attribute; make that first call before any stream capture.
 *   - All calls share the scratch: calls that overlap on the GPU race; serialise them.
 *   - It calls no cudaMalloc, cudaFree or allocating library routine.
 * hb_static_last_error returns the calling thread's last message; hb_static_status copies
 * back (blocking) and clears the device-side status words of the static launches. */
hb_status hb_matmul_skinny_static(const void* A, const void* B, void* C, int64_t M, int64_t N,
                                  int64_t K, int32_t device, void* cuda_stream);
const char* hb_static_last_error(void);
hb_status hb_static_status(int32_t device, int32_t* out4);

/* ---- model-IR attention node --------------------------------------------------------
 * O = softmax(scale * Q K^T + causal mask) V per (batch, head).  Tensors are
 * [batch, seq, heads, head_dim] bf16 (token-major); n_q_heads must be a multiple of
 * n_kv_heads (grouped-query attention).  fp32 scores, fp32 running max/sum, P rounded
 * to bf16 before the PV product.  `lse` (optional, fp32 [batch, heads, seq]) receives
 * log-sum-exp of the scaled scores.  No reference counterpart. */
typedef struct hb_attn_opts {
  int32_t causal;
  float scale;
  void* lse;
  int32_t config_id;
} hb_attn_opts;
hb_status hb_attention(hb_ctx* ctx, const hb_tensor* Q, const hb_tensor* K,
                       const hb_tensor* V, hb_tensor* O, const hb_attn_opts* opts);
hb_status hb_attention_host(hb_ctx* ctx, const void* Q, const void* K, const void* V, void* O,
                            int64_t batch, int64_t seq, int64_t n_q_heads,
                            int64_t n_kv_heads, int64_t head_dim, int32_t causal,
                            float scale);

/* ---- decode-shaped path: one new token per sequence against a key/value cache --------
 * Cache: kv_cache[2 * batch, s_max, n_kv_heads, 128] bf16 -- keys in the first `batch`
 * entries, values in the second, token-major like the attention node's tensors.  `qkv` is
 * the new token's projection, one row per sequence: q heads, then k heads, then v heads
 * (row_stride elements per row).  `pos_dev` is a DEVICE int32: the position of the new token
 * (the cache then holds pos + 1 tokens), shared by all sequences; keeping it on the device
 * makes every step's launches identical, so a planned step can be captured and replayed.
 * No reference counterpart (the reference has no attention at all).
 *   hb_rope_append       rotate-half RoPE of the q and k heads at *pos_dev, in place (same
 *                        angles as hb_rope: theta_i = base^(-2i/128), formed in double), and
 *                        append of the rotated k heads and the v heads to the cache.  A full
 *                        cache (*pos_dev >= s_max) writes nothing and makes the next hb_sync
 *                        return HB_ERR_INVALID.
 *   hb_attention_decode  out[batch, n_q_heads * 128] = softmax(scale * q K^T) V over cache
 *                        positions 0..*pos_dev, fp32 scores / max / sum; grouped-query heads
 *                        share one pass over their KV head.  The positions are split over
 *                        CTAs (len_hint: expected length, used only to size the splits; 0 =
 *                        s_max) and merged in a fixed order: bit-identical run to run.
 *   hb_advance_pos       *pos_dev += n. */
hb_status hb_rope_append(hb_ctx* ctx, void* qkv, int64_t row_stride, void* kv_cache,
                         const int32_t* pos_dev, int64_t batch, int64_t n_q_heads,
                         int64_t n_kv_heads, int64_t head_dim, int64_t s_max, float base);
hb_status hb_attention_decode(hb_ctx* ctx, const void* qkv, int64_t row_stride,
                              const void* kv_cache, const int32_t* pos_dev, void* out,
                              int64_t batch, int64_t n_q_heads, int64_t n_kv_heads,
                              int64_t head_dim, int64_t s_max, int64_t len_hint, float scale);
hb_status hb_advance_pos(hb_ctx* ctx, int32_t* pos_dev, int32_t n);

/* ---- glue operators the decoder / MLP configurations put on the path ------------- */
/* y = x * rsqrt(mean(x^2) + eps) * gain; rows x cols bf16, gain bf16[cols]. If
 * `residual_inout` is non-NULL it is first updated in place: residual += x, and the
 * norm is taken of the updated residual (fused residual add). */
hb_status hb_rmsnorm(hb_ctx* ctx, const void* x, const void* gain, void* y,
                     void* residual_inout, int64_t rows, int64_t cols, float eps);
/* Rotate-half RoPE in place over x[tokens, heads, head_dim]; position of token t is
 * pos0 + (t % seq). theta_i = base^(-2i/head_dim). */
hb_status hb_rope(hb_ctx* ctx, void* x, int64_t tokens, int64_t seq, int64_t heads,
                  int64_t head_dim, int64_t row_stride, float base, int64_t pos0);
/* out[t, :] = table[ids[t], :] (bit-exact gather). */
hb_status hb_embedding(hb_ctx* ctx, const void* table, const int32_t* ids, void* out,
                       int64_t tokens, int64_t vocab, int64_t dim);
/* out[r, j] = silu(x[r, j]) * x[r, half + j]  for x[rows, 2*half] bf16. */
hb_status hb_swiglu(hb_ctx* ctx, const void* x, void* out, int64_t rows, int64_t half);
hb_status hb_gelu(hb_ctx* ctx, const void* x, void* y, int64_t n);
/* dx = dy * gelu'(x) (erf-exact derivative). */
hb_status hb_gelu_backward(hb_ctx* ctx, const void* x, const void* dy, void* dx, int64_t n);
hb_status hb_add(hb_ctx* ctx, const void* a, const void* b, void* out, int64_t n);
/* Mean-squared error over n bf16 elements: *loss (device fp32) = mean((y - target)^2),
 * dy = 2 (y - target) / n (bf16).  Partial sums are added in a fixed order. */
hb_status hb_mse(hb_ctx* ctx, const void* y, const void* target, void* dy, float* loss, int64_t n);
/* One bias-corrected Adam step (no weight decay) on fp32 master weights w and moments m, v
 * from a bf16 gradient scaled by grad_scale; also refreshes the bf16 copy of the weights.
 * step counts from 1. */
hb_status hb_adam_step(hb_ctx* ctx, float* w, float* m, float* v, const void* grad_bf16,
                       void* w_bf16, int64_t n, float lr, float beta1, float beta2, float eps,
                       int64_t step, float grad_scale);
/* The same update enqueued on the context's side stream behind everything queued so far
 * (hb_side_join makes the main stream wait for it): the HBM-bound optimizer step of a layer
 * runs under the tensor-bound backward products of the layers still to come. */
hb_status hb_adam_step_async(hb_ctx* ctx, float* w, float* m, float* v, const void* grad_bf16,
                       void* w_bf16, int64_t n, float lr, float beta1, float beta2, float eps,
                       int64_t step, float grad_scale);
/* argmax over the last dimension, first index wins ties (bit-exact). */
hb_status hb_argmax(hb_ctx* ctx, const void* x, int32_t* out, int64_t rows, int64_t cols);

/* ---- model-IR collective node ----------------------------------------------------
 * Sum-allreduce of `count` bf16/f32 elements in place across the ranks of the
 * communicator bound to `ctx`.  HB_AR_NCCL enqueues ncclAllReduce on the stream;
 * HB_AR_P2P runs this library's two-shot kernel over peer-mapped buffers (plain peer
 * loads and stores, bounded flag waits). No reference counterpart. */
enum { HB_AR_AUTO = 0, HB_AR_NCCL = 1, HB_AR_P2P = 2, HB_AR_NVLS = 3 };
#define HB_UNIQUE_ID_BYTES 128
#define HB_IPC_HANDLE_BYTES 64
hb_status hb_comm_unique_id(void* id_out /* HB_UNIQUE_ID_BYTES */);
hb_status hb_comm_init_rank(hb_ctx* ctx, int32_t world, int32_t rank, const void* unique_id);
hb_status hb_comm_destroy(hb_ctx* ctx);
/* P2P set-up: each rank allocates a symmetric buffer, exports its handle, exchanges
 * handles out of band (any host channel) and opens its peers'. */
hb_status hb_p2p_alloc(hb_ctx* ctx, size_t bytes, void** dev_ptr, void* handle_out);
hb_status hb_p2p_attach(hb_ctx* ctx, int32_t world, int32_t rank, const void* all_handles,
                        size_t bytes);
/* Alternative to hb_p2p_alloc/attach for callers that already own a symmetric buffer
 * (and, optionally, its NVSwitch multicast mapping, which enables HB_AR_NVLS: the sum is
 * taken inside the switch with multimem.ld_reduce / multimem.st).  Each rank's buffer holds
 * `bytes` of payload, rounded up to 256, followed by hb_p2p_flag_bytes() zeroed bytes. */
size_t hb_p2p_flag_bytes(void);
hb_status hb_p2p_attach_external(hb_ctx* ctx, int32_t world, int32_t rank,
                                 const void* const* peer_ptrs, void* multicast_ptr, size_t bytes);
hb_status hb_all_reduce(hb_ctx* ctx, void* data, int64_t count, int32_t dtype, int32_t algo);
/* Every cross-GPU flag wait inside the collective kernels polls at most `polls` times
 * (default 2^24, a few seconds) before the kernel records HB_ERR_TIMEOUT, skips its work and
 * returns; hb_sync then reports the time-out and the context stays usable.  A host that has
 * its own failure detector sets a smaller limit; all ranks should use the same one.
 * No reference counterpart (the reference reports failures as `Result` values,
 * `src/lib/error.ml:18-26`, and never waits on a device). */
hb_status hb_comm_set_wait_limit(hb_ctx* ctx, uint32_t polls);
/* Kernel form of hb_all_reduce_norm.  fused_form 1: one CTA per row, the faster form when the
 * collective has the GPU to itself; 2: one warp per row on at most `fused_ctas` CTAs (0 = one
 * per SM), small enough to run beside a GEMM on the same SMs, the form for collectives that
 * overlap compute; 0 (default): form 1 on the context's own stream, form 2 on its side stream.
 * The results are the same bits in every form.  Every rank must make the same choice.
 * No reference counterpart. */
hb_status hb_comm_configure(hb_ctx* ctx, int32_t fused_form, int32_t fused_ctas);
/* Overlap: hb_all_reduce_async enqueues the same allreduce on the context's high-priority
 * side stream, ordered after everything already queued on the main stream, and returns;
 * hb_side_join makes the main stream wait for the side stream.  Kernels queued between the
 * two calls must not touch the tensor being reduced. */
hb_status hb_all_reduce_async(hb_ctx* ctx, void* data, int64_t count, int32_t dtype, int32_t algo);
hb_status hb_side_join(hb_ctx* ctx);
/* Fused collective for the tensor-parallel block: reduce-scatter of the row-parallel
 * partial products, residual add and RMSNorm on this rank's rows/world rows, all-gather of
 * the normalised rows -- one kernel over peer memory (HB_AR_P2P) or through NVSwitch
 * (HB_AR_NVLS), bf16.  `partial` and `out` are [rows, cols] inside the symmetric buffer;
 * `residual_in` / `residual_out` are local [rows, cols] of which only this rank's rows are
 * read / written: residual_out = bf16(residual_in + bf16(sum of partials)).
 * mode 0: out = rmsnorm(residual_out) * gain; mode 1: out = residual_out (final gather).
 * Adding 2 to `mode` makes the call publish one "rows ready" word per block of gathered rows
 * as the rows land, which is what hb_matmul_gathered waits for (warp-per-row form only). */
hb_status hb_all_reduce_norm(hb_ctx* ctx, const void* partial, const void* gain,
                             const void* residual_in, void* residual_out, void* out,
                             int64_t rows, int64_t cols, float eps, int32_t mode, int32_t algo);

/* ---- model-IR executor: node list, memory planner, launcher --------------------------
 * A graph is an ordered list of operator nodes over tensor ids.  `hb_graph_plan` computes
 * each planner-owned tensor's lifetime and packs them into one arena (and the tensors
 * flagged HB_T_SYMMETRIC into the peer-mapped buffer, when the context has one, so that
 * allreduce runs in place over NVLink); `hb_graph_run` enqueues every node on the
 * context's stream.  Shape taken from the reference's only program walker, a list of
 * variant-tagged definitions dispatched in order (`lift_defs_exn`, tree.ml:786-811). */
typedef struct hb_graph hb_graph;
enum {
  HB_NODE_MATMUL = 0,      /* in: A, B, [residual]      iparam: epilogue, config_id, gathered (1: A is the
                              output of the preceding all_reduce_norm node; hb_matmul_gathered)   */
  HB_NODE_ATTENTION = 1,   /* in: Q, K, V, [lse]        iparam: causal        fparam: scale   */
  HB_NODE_ALL_REDUCE = 2,  /* in place on `out`         iparam: algorithm                     */
  HB_NODE_RMSNORM = 3,     /* in: x, gain, [residual]                         fparam: eps     */
  HB_NODE_ROPE = 4,        /* in place on `out`         iparam: seq, heads, head_dim, pos0; fparam: base */
  HB_NODE_EMBEDDING = 5,   /* in: table, ids */
  HB_NODE_SWIGLU = 6,      /* in: x */
  HB_NODE_GELU = 7,        /* in: x */
  HB_NODE_ADD = 8,         /* in: a, b */
  HB_NODE_ARGMAX = 9,      /* in: x */
  HB_NODE_AR_NORM = 10,    /* in: partial, [gain], residual_in, residual_out (written); out: normalised
                              or gathered rows   iparam: mode, algorithm   fparam: eps */
  HB_NODE_ROPE_APPEND = 11,  /* in: qkv [batch, row] (rotated in place), pos (i32[1]); out: kv cache
                                [2*batch, s_max, kv_heads, 128]   iparam: q heads, kv heads   fparam: base */
  HB_NODE_ATTN_DECODE = 12,  /* in: qkv, kv cache, pos; out: [batch, q_heads*128]
                                iparam: q heads, kv heads, len_hint   fparam: scale */
  HB_NODE_ADVANCE = 13       /* in place on `out` (i32[1])   iparam: increment */
};
enum { HB_T_SYMMETRIC = 1 };
typedef struct hb_node {
  int32_t kind;
  int32_t in[4];           /* tensor ids, -1 where unused */
  int32_t out;
  int32_t iparam[4];
  float fparam[2];
  int32_t stream;          /* 0: the context's stream; 1: its side stream (runs concurrently;
                              the executor orders conflicting nodes with events).  Only
                              HB_NODE_ALL_REDUCE and HB_NODE_AR_NORM nodes may use stream 1:
                              compute nodes share per-context scratch that the byte-range
                              analysis does not see */
} hb_node;
hb_status hb_graph_create(hb_ctx* ctx, hb_graph** out);
hb_status hb_graph_destroy(hb_graph* g);
/* Caller-owned tensor (weights, inputs, outputs). */
hb_status hb_graph_input(hb_graph* g, const hb_tensor* t, int32_t* id);
/* Planner-owned contiguous tensor. */
hb_status hb_graph_temp(hb_graph* g, int32_t dtype, int32_t rank, const int64_t* shape,
                        int32_t flags, int32_t* id);
/* View of another tensor: element offset, shape and strides (elements). */
hb_status hb_graph_view(hb_graph* g, int32_t base, int64_t offset, int32_t rank,
                        const int64_t* shape, const int64_t* stride, int32_t* id);
hb_status hb_graph_add(hb_graph* g, const hb_node* node);
hb_status hb_graph_plan(hb_graph* g, size_t* arena_bytes, size_t* symmetric_bytes);
/* The planner's placement rule on its own (host arithmetic only, needs no context or GPU):
 * `n` buffers of `bytes[i]` alive over node indices [first[i], last[i]] are packed largest
 * first, each at the lowest 256-byte-aligned offset free during its lifetime.  No reference
 * counterpart (the reference allocates nothing on a device). */
hb_status hb_plan_arena(int32_t n, const size_t* bytes, const int32_t* first, const int32_t* last,
                        size_t* offsets, size_t* total);
hb_status hb_graph_run(hb_graph* g);
/* Replay: hb_graph_capture records one run of the planned graph (both streams and the event
 * edges between them) into a CUDA graph; hb_graph_replay enqueues that whole step on the
 * context's stream with one call.  The graph must have run once through hb_graph_run since it
 * was planned (scratch buffers reach their size on first use); everything read from the host --
 * addresses, shapes, configuration choices -- is frozen at capture time, so per-step values
 * must live in device memory (the decode position does); hb_graph_plan drops the capture.
 * Graphs with collective nodes on more than one rank are refused (HB_ERR_UNSUPPORTED).
 * No reference counterpart. */
hb_status hb_graph_capture(hb_graph* g);
hb_status hb_graph_replay(hb_graph* g);
/* One run with a CUDA event between nodes: ms[i] = device time of node i (first n nodes). */
hb_status hb_graph_run_timed(hb_graph* g, float* ms, int32_t n);
hb_status hb_graph_describe(hb_graph* g, char* buf, size_t len);
hb_status hb_graph_tensor_ptr(hb_graph* g, int32_t id, void** ptr);

/* ---- autotune entry point ----------------------------------------------------------
 * Searches the configurations of one operator for one problem shape by timing each
 * candidate on the device, records the winner in the context's cache, and can persist the
 * cache as text.  No reference counterpart.
 *   matmul (M > 64)   tile N (64 / 128 / 256), cluster shape (one CTA per 128-row tile or a CTA
 *                     pair per 256-row tile), ring depth, K-block width (64 or 128 per ring
 *                     stage) and raster order, each varied on its own;
 *   matmul (M <= 64)  the stream-K kernel: persistent grid and k-blocks per ring stage;
 *   attention         one work unit per CTA or the persistent work queue.
 * The text cache writes a choice by its properties and keys it by operator, shape, layout,
 * epilogue, SM count and GPU name (hb_tune_cache_save / _load; version-1 files are read). */
enum { HB_OP_MATMUL = 0, HB_OP_ATTENTION = 1 };
enum { HB_TUNE_CACHED = 0, HB_TUNE_SEARCH = 1 };
typedef struct hb_op_desc {
  int32_t op;              /* HB_OP_* */
  int32_t dtype;
  int64_t m, n, k;         /* matmul: M,N,K; attention: batch, seq, head_dim (128) */
  int32_t layout;          /* matmul: bit0 A is M-major, bit1 B is N-major; attention: 1 = causal */
  int32_t epilogue;        /* matmul: HB_EPI_*; attention: n_q_heads << 16 | n_kv_heads */
} hb_op_desc;
typedef struct hb_tune_result {
  int32_t config_id;       /* matmul: index for hb_matmul_opts.config_id (-1: stream-K kernel);
                              attention: 0 one unit per CTA, 1 persistent (hb_attn_opts.config_id) */
  int32_t tile_m, tile_n, tile_k, stages, cluster, raster_group;
  int32_t split_k;         /* stream-K kernel: persistent grid (K ranges in flight); else 1 */
  float ms;
  float tflops;
} hb_tune_result;
hb_status hb_autotune(hb_ctx* ctx, const hb_op_desc* desc, int32_t mode, hb_tune_result* out);
hb_status hb_tune_cache_load(hb_ctx* ctx, const char* path);
hb_status hb_tune_cache_save(hb_ctx* ctx, const char* path);
int32_t hb_matmul_config_count(void);
hb_status hb_matmul_config_info(int32_t config_id, hb_tune_result* out);
/* Where the dispatcher sends a bf16 matmul when the autotune cache has no entry for it
 * (host arithmetic only, needs no context or GPU): `kernel` 0 = one-CTA tile kernel,
 * 1 = CTA-pair 256 x 256 tile kernel, 2 = stream-K kernel for M <= 64; `config_id` for
 * kernels 0 and 1; for kernel 2 the persistent grid, the column tiles, the most K ranges
 * that can share a tile and the fp32 scratch the launch uses. */
typedef struct hb_matmul_route {
  int32_t kernel;
  int32_t config_id;
  int32_t grid;
  int32_t tiles;
  int32_t max_segments;
  int64_t scratch_bytes;
} hb_matmul_route;
hb_status hb_matmul_default_route(int32_t sm_count, const hb_op_desc* desc, hb_matmul_route* out);

#ifdef __cplusplus
}
#endif
#endif /* HABU_B200_H */
