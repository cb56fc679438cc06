// Context, memory, error plumbing and the matmul node's host side (validation, layout
// decoding, configuration choice) of libhabu_b200.so.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include "hb_internal.h"

hb_status hb_fail(hb_ctx* ctx, hb_status code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf;
  return code;
}

hb_status hb_check_cuda(hb_ctx* ctx, cudaError_t e, const char* what) {
  if (e == cudaSuccess) return HB_OK;
  return hb_fail(ctx, HB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

extern "C" hb_status hb_ctx_create(int32_t device, hb_ctx** out) {
  if (!out) return HB_ERR_INVALID;
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || device < 0 || device >= n) return HB_ERR_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return HB_ERR_CUDA;
  if (prop.major != 10) return HB_ERR_UNSUPPORTED;  // kernels are sm_100a only
  if (cudaSetDevice(device) != cudaSuccess) return HB_ERR_CUDA;
  hb_ctx* ctx = new hb_ctx();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->gpu_name = prop.name;
  for (char& c : ctx->gpu_name)
    if (c == ' ' || c == '\t') c = '_';
  if (cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc(&ctx->d_status, 16 * sizeof(int32_t)) != cudaSuccess ||     // 4 status words, 4 spare, 8 work counters
      cudaMemset(ctx->d_status, 0, 16 * sizeof(int32_t)) != cudaSuccess ||
      cudaMalloc(&ctx->d_tickets, HB_MAX_SPLITK_TILES * sizeof(int)) != cudaSuccess ||
      cudaMemset(ctx->d_tickets, 0, HB_MAX_SPLITK_TILES * sizeof(int)) != cudaSuccess ||
      cudaMallocHost(&ctx->h_status, 4 * sizeof(int32_t)) != cudaSuccess) {
    delete ctx;
    return HB_ERR_CUDA;
  }
  ctx->stream = ctx->own_stream;
  *out = ctx;
  return HB_OK;
}

extern "C" hb_status hb_ctx_destroy(hb_ctx* ctx) {
  if (!ctx) return HB_ERR_INVALID;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  hb_comm_destroy(ctx);
  for (void* p : ctx->allocations) cudaFree(p);
  for (void* p : ctx->scratch)
    if (p) cudaFree(p);
  if (ctx->rope_table) cudaFree(ctx->rope_table);
  if (ctx->d_tickets) cudaFree(ctx->d_tickets);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->h_status) cudaFreeHost(ctx->h_status);
  for (cudaEvent_t e : ctx->event_pool) cudaEventDestroy(e);
  if (ctx->h2d_stream) cudaStreamDestroy(ctx->h2d_stream);
  if (ctx->d2h_stream) cudaStreamDestroy(ctx->d2h_stream);
  if (ctx->side_event) cudaEventDestroy(ctx->side_event);
  if (ctx->side_stream) cudaStreamDestroy(ctx->side_stream);
  if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
  delete ctx;
  return HB_OK;
}

extern "C" hb_status hb_ctx_set_stream(hb_ctx* ctx, void* cuda_stream) {
  if (!ctx) return HB_ERR_INVALID;
  ctx->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : ctx->own_stream;
  return HB_OK;
}

extern "C" const char* hb_last_error_string(hb_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }

extern "C" hb_status hb_alloc(hb_ctx* ctx, size_t bytes, void** dev_ptr) {
  if (!ctx || !dev_ptr) return HB_ERR_INVALID;
  HB_CUDA(ctx, cudaSetDevice(ctx->device));
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    return hb_fail(ctx, HB_ERR_NOMEM, "hb_alloc: out of device memory (%zu bytes)", bytes);
  }
  if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaMalloc");
  ctx->allocations.push_back(p);
  *dev_ptr = p;
  return HB_OK;
}

extern "C" hb_status hb_free(hb_ctx* ctx, void* dev_ptr) {
  if (!ctx) return HB_ERR_INVALID;
  if (!dev_ptr) return HB_OK;
  for (size_t i = 0; i < ctx->allocations.size(); ++i) {
    if (ctx->allocations[i] == dev_ptr) {
      ctx->allocations.erase(ctx->allocations.begin() + i);
      HB_CUDA(ctx, cudaSetDevice(ctx->device));
      HB_CUDA(ctx, cudaFree(dev_ptr));
      return HB_OK;
    }
  }
  return hb_fail(ctx, HB_ERR_NOT_FOUND, "hb_free: pointer was not allocated by this context");
}

extern "C" hb_status hb_upload(hb_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes) {
  if (!ctx || (!dst_dev && bytes) || (!src_host && bytes)) return HB_ERR_INVALID;
  HB_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return HB_OK;
}

extern "C" hb_status hb_download(hb_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes) {
  if (!ctx || (!dst_host && bytes) || (!src_dev && bytes)) return HB_ERR_INVALID;
  HB_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return HB_OK;
}

extern "C" hb_status hb_sync(hb_ctx* ctx) {
  if (!ctx) return HB_ERR_INVALID;
  HB_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, 4 * sizeof(int32_t),
                               cudaMemcpyDeviceToHost, ctx->stream));
  HB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->h_status[0] != 0) {
    const int code = ctx->h_status[0], tag = ctx->h_status[1], detail = ctx->h_status[2];
    cudaMemsetAsync(ctx->d_status, 0, 4 * sizeof(int32_t), ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    return hb_fail(ctx, code, "device-side status %d from kernel tag %d (detail %d)", code, tag,
                   detail);
  }
  return HB_OK;
}

extern "C" int64_t hb_launch_count(hb_ctx* ctx) { return ctx ? ctx->launches : -1; }
extern "C" int32_t hb_sm_count(hb_ctx* ctx) { return ctx ? ctx->sm_count : -1; }

// Waits for every stream the context may have work on (the stream in use, its own stream and
// the side stream): called before context-owned memory is freed, because a kernel queued on
// the OTHER stream of a two-stream graph may still be using it.
hb_status hb_quiesce(hb_ctx* ctx) {
  HB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->own_stream && ctx->own_stream != ctx->stream) HB_CUDA(ctx, cudaStreamSynchronize(ctx->own_stream));
  if (ctx->side_stream && ctx->side_stream != ctx->stream) HB_CUDA(ctx, cudaStreamSynchronize(ctx->side_stream));
  return HB_OK;
}

hb_status hb_get_scratch(hb_ctx* ctx, int slot, size_t bytes, void** out) {
  if (bytes > ctx->scratch_bytes[slot]) {
    HB_CUDA(ctx, cudaSetDevice(ctx->device));
    if (ctx->scratch[slot]) {
      hb_status qs = hb_quiesce(ctx);
      if (qs != HB_OK) return qs;
      HB_CUDA(ctx, cudaFree(ctx->scratch[slot]));
      ctx->scratch[slot] = nullptr;
      ctx->scratch_bytes[slot] = 0;
    }
    size_t want = bytes < (size_t(1) << 20) ? (size_t(1) << 20) : bytes;
    cudaError_t e = cudaMalloc(&ctx->scratch[slot], want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return hb_fail(ctx, HB_ERR_NOMEM, "scratch: cannot allocate %zu bytes", want);
    }
    ctx->scratch_bytes[slot] = want;
  }
  *out = ctx->scratch[slot];
  return HB_OK;
}

// ------------------------------------------------------------------ tensor maps
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled get_encode_fn() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(p);
  });
  return fn;
}

// Encoded maps are kept per context, keyed by everything that goes into the encoding: a
// graph replays the same few dozen (buffer, shape, box) combinations every step, and three
// driver calls per launch are host time inside every launch gap.  The descriptor holds the
// address, not the data, so a cached map stays valid for as long as the same address is used
// with the same geometry.
struct hb_tmap_key {
  const void* base;
  uint64_t dims[5], strides[4];
  uint32_t box[5];
  int32_t dt, rank, swizzle;
  bool operator==(const hb_tmap_key& o) const { return memcmp(this, &o, sizeof(*this)) == 0; }
};

hb_status hb_make_tensor_map(hb_ctx* ctx, CUtensorMap* out, CUtensorMapDataType dt, int rank,
                             const void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                             const uint32_t* box, CUtensorMapSwizzle swizzle) {
  PFN_encodeTiled fn = get_encode_fn();
  if (!fn) return hb_fail(ctx, HB_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  if (rank < 1 || rank > 5) return hb_fail(ctx, HB_ERR_INVALID, "tensor map rank %d", rank);
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
    return hb_fail(ctx, HB_ERR_INVALID, "tensor base address must be 16-byte aligned");
  for (int i = 0; i + 1 < rank; ++i)
    if (strides_bytes[i] & 15)
      return hb_fail(ctx, HB_ERR_INVALID,
                     "tensor stride %d (%llu bytes) must be a multiple of 16 bytes", i + 1,
                     (unsigned long long)strides_bytes[i]);
  hb_tmap_key key;
  memset(&key, 0, sizeof(key));
  key.base = base; key.dt = (int32_t)dt; key.rank = rank; key.swizzle = (int32_t)swizzle;
  for (int i = 0; i < rank; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; if (i + 1 < rank) key.strides[i] = strides_bytes[i]; }
  uint64_t h = 1469598103934665603ull;                   // FNV-1a over the key
  for (size_t i = 0; i < sizeof(key); ++i) { h ^= reinterpret_cast<const unsigned char*>(&key)[i]; h *= 1099511628211ull; }
  if (ctx) {
    auto range = ctx->tmap_cache.equal_range(h);
    for (auto it = range.first; it != range.second; ++it)
      if (memcmp(it->second.key, &key, sizeof(key)) == 0) { memcpy(out, it->second.map, sizeof(CUtensorMap)); return HB_OK; }
  }
  cuuint64_t gdims[5];
  cuuint64_t gstr[5];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstr, gbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return hb_fail(ctx, HB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  if (ctx) {
    if (ctx->tmap_cache.size() >= 8192) ctx->tmap_cache.clear();      // bounded: start over rather than grow
    hb_tmap_entry e;
    static_assert(sizeof(e.key) >= sizeof(hb_tmap_key), "tensor-map cache key storage");
    memset(&e, 0, sizeof(e));
    memcpy(e.key, &key, sizeof(key));
    memcpy(e.map, out, sizeof(CUtensorMap));
    ctx->tmap_cache.emplace(h, e);
  }
  return HB_OK;
}

// ------------------------------------------------------------------ matmul node
static hb_status decode_matmul(hb_ctx* ctx, const hb_tensor* A, const hb_tensor* B,
                               const hb_tensor* C, const hb_matmul_opts* opts, hb_gemm_args* g) {
  if (!A || !B || !C) return hb_fail(ctx, HB_ERR_INVALID, "matmul: null tensor");
  if (A->rank != 2 || B->rank != 2 || C->rank != 2)
    return hb_fail(ctx, HB_ERR_INVALID, "matmul: tensors must have rank 2");
  if (!A->ptr || !B->ptr || !C->ptr) return hb_fail(ctx, HB_ERR_INVALID, "matmul: null data pointer");
  if (A->dtype != B->dtype || A->dtype != C->dtype)
    return hb_fail(ctx, HB_ERR_INVALID, "matmul: dtypes of A, B and C must agree");
  if (A->dtype != HB_BF16 && A->dtype != HB_F32)
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "matmul: dtype %d is not supported", A->dtype);
  const int64_t M = A->shape[0], K = A->shape[1], N = B->shape[1];
  const int epi = opts ? (opts->epilogue & 0xff) : HB_EPI_NONE;
  const bool weights_b = opts && (opts->epilogue & HB_MATMUL_WEIGHTS_B);
  if (epi < HB_EPI_NONE || epi > HB_EPI_RESIDUAL)
    return hb_fail(ctx, HB_ERR_INVALID, "matmul: unknown epilogue %d", epi);
  const int64_t NC = (epi == HB_EPI_SWIGLU) ? N / 2 : N;
  if (B->shape[0] != K)
    return hb_fail(ctx, HB_ERR_INVALID, "matmul: inner dimensions differ (A is %lld x %lld, B is %lld x %lld)",
                   (long long)M, (long long)K, (long long)B->shape[0], (long long)N);
  if (C->shape[0] != M || C->shape[1] != NC)
    return hb_fail(ctx, HB_ERR_INVALID, "matmul: C must be %lld x %lld", (long long)M, (long long)NC);
  if (M <= 0 || N <= 0 || K <= 0) return hb_fail(ctx, HB_ERR_INVALID, "matmul: empty dimension");
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "matmul: dimension exceeds 2^31-1");
  if (epi == HB_EPI_SWIGLU && (N & 1))
    return hb_fail(ctx, HB_ERR_INVALID, "matmul: swiglu epilogue needs an even N");
  if (C->stride[1] != 1) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "matmul: C must be row-major");
  memset(g, 0, sizeof(*g));
  g->A = A->ptr; g->B = B->ptr; g->C = C->ptr;
  g->M = M; g->N = N; g->K = K;
  g->ldc = C->stride[0];
  if (g->ldc < NC) return hb_fail(ctx, HB_ERR_INVALID, "matmul: C row stride smaller than its width");
  if (A->stride[1] == 1 && (A->stride[0] >= K)) { g->a_mn_major = 0; g->lda = A->stride[0]; }
  else if (A->stride[0] == 1 && A->stride[1] >= M) { g->a_mn_major = 1; g->lda = A->stride[1]; }
  else return hb_fail(ctx, HB_ERR_UNSUPPORTED, "matmul: A must be contiguous along K or along M");
  if (B->stride[0] == 1 && B->stride[1] >= K) { g->b_mn_major = 0; g->ldb = B->stride[1]; }
  else if (B->stride[1] == 1 && B->stride[0] >= N) { g->b_mn_major = 1; g->ldb = B->stride[0]; }
  else return hb_fail(ctx, HB_ERR_UNSUPPORTED, "matmul: B must be contiguous along K or along N");
  g->epilogue = epi;
  g->b_is_weights = weights_b ? 1 : 0;
  if (epi == HB_EPI_RESIDUAL) {
    if (!opts->residual) return hb_fail(ctx, HB_ERR_INVALID, "matmul: residual epilogue without a residual");
    g->residual = opts->residual;
    g->ldr = opts->residual_ld ? opts->residual_ld : N;
  }
  return HB_OK;
}

extern "C" hb_status hb_matmul(hb_ctx* ctx, const hb_tensor* A, const hb_tensor* B, hb_tensor* C,
                               const hb_matmul_opts* opts) {
  if (!ctx) return HB_ERR_INVALID;
  hb_gemm_args g;
  hb_status st = decode_matmul(ctx, A, B, C, opts, &g);
  if (st != HB_OK) return st;
  if (A->dtype == HB_F32) {
    if (g.epilogue != HB_EPI_NONE)
      return hb_fail(ctx, HB_ERR_UNSUPPORTED, "matmul: fp32 path has no fused epilogue");
    return hb_launch_gemm_f32(ctx, g);
  }
  // TMA needs 16-byte aligned bases and row pitches.
  if ((g.lda & 7) || (g.ldb & 7))
    return hb_fail(ctx, HB_ERR_UNSUPPORTED,
                   "matmul: bf16 operand leading dimensions must be multiples of 8 elements");
  if (!(opts && opts->config_id >= 0) && hb_gemm_skinny_applicable(g)) return hb_launch_gemm_skinny(ctx, g);
  int cfg = (opts && opts->config_id >= 0) ? opts->config_id : hb_gemm_pick_config(ctx, g);
  return hb_launch_gemm_bf16(ctx, g, cfg);
}

// Matmul whose A is the gathered output of the hb_all_reduce_norm call enqueued just before it
// (on any stream of this context).  The collective publishes one "rows ready" word per block of
// rows as the rows land; this kernel's loader waits for the word of a block before its first
// load from it and visits the row blocks owner by owner, this rank's own rows first, so the
// product of the rows that have arrived runs while the rest are still crossing NVLink.  It may
// therefore be enqueued on a stream that does NOT wait for the collective.
extern "C" hb_status hb_matmul_gathered(hb_ctx* ctx, const hb_tensor* A, const hb_tensor* B, hb_tensor* C,
                                        const hb_matmul_opts* opts) {
  if (!ctx) return HB_ERR_INVALID;
  if (ctx->world <= 1 || ctx->p2p.world <= 1) return hb_matmul(ctx, A, B, C, opts);
  hb_gemm_args g;
  hb_status st = decode_matmul(ctx, A, B, C, opts, &g);
  if (st != HB_OK) return st;
  const hb_p2p_state& s = ctx->p2p;
  if (A->dtype != HB_BF16 || g.a_mn_major || (g.lda & 7) || (g.ldb & 7) || hb_gemm_skinny_applicable(g))
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "matmul_gathered: needs a row-major bf16 A with more than 64 rows");
  if (s.ready_rows <= 0 || s.ready_out != A->ptr || s.ready_total_rows != g.M)
    return hb_fail(ctx, HB_ERR_INVALID,
                   "matmul_gathered: A is not the output of the hb_all_reduce_norm enqueued before this call "
                   "(or that call published no ready words)");
  g.ready = reinterpret_cast<const uint32_t*>(static_cast<const char*>(s.local) + s.bytes + hb_p2p_ready_offset());
  g.ready_epoch = s.ready_epoch;
  g.ready_spin = s.spin_limit;
  g.ready_rows = s.ready_rows;
  g.perm_world = s.world;
  g.perm_rank = s.rank;
  const int cfg = (opts && opts->config_id >= 0) ? opts->config_id : hb_gemm_pick_config(ctx, g);
  return hb_launch_gemm_bf16(ctx, g, cfg);
}

hb_status hb_host_pipe(hb_ctx* ctx, int n, cudaEvent_t** events) {
  HB_CUDA(ctx, cudaSetDevice(ctx->device));
  if (!ctx->h2d_stream) HB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking));
  if (!ctx->d2h_stream) HB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking));
  while ((int)ctx->event_pool.size() < n) {
    cudaEvent_t e;
    HB_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    ctx->event_pool.push_back(e);
  }
  *events = ctx->event_pool.data();
  return HB_OK;
}

// Host-buffer matmul.  Large bf16 products are pipelined in row chunks over three streams:
// copy-in (B, then the A chunks), compute (one matmul per chunk as soon as its rows have
// landed) and copy-out (each C chunk as soon as it is computed), so the PCIe transfers in
// both directions run under each other and under the kernels.
extern "C" hb_status hb_matmul_host(hb_ctx* ctx, const void* A_host, const void* B_host, void* C_host,
                                    int64_t M, int64_t N, int64_t K, int32_t dtype) {
  if (!ctx) return HB_ERR_INVALID;
  if (!A_host || !B_host || !C_host) return hb_fail(ctx, HB_ERR_INVALID, "matmul_host: null buffer");
  if (M <= 0 || N <= 0 || K <= 0) return hb_fail(ctx, HB_ERR_INVALID, "matmul_host: empty dimension");
  const size_t es = dtype == HB_BF16 ? 2 : dtype == HB_F32 ? 4 : 0;
  if (!es) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "matmul_host: dtype %d", dtype);
  const size_t a_b = (size_t)M * K * es, b_b = (size_t)N * K * es, c_b = (size_t)M * N * es;
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  void* base = nullptr;
  hb_status st = hb_get_scratch(ctx, HB_SCRATCH_STAGING, up(a_b) + up(b_b) + up(c_b), &base);
  if (st != HB_OK) return st;
  char* dA = static_cast<char*>(base);
  char* dB = dA + up(a_b);
  char* dC = dB + up(b_b);
  // Row chunks of 1024 (4 to 8 of them): what is left after the last byte of A has landed is one
  // chunk's product and one chunk's copy-out, so smaller chunks shorten the tail of the call.
  // Measured at 8192^3: 6.04 ms with 4 chunks, 5.90 with 8, 6.17 with 16 (512-row products fill
  // less than one wave of tile pairs, and twice as many copy-outs cut into the copy-in).
  int chunks = (dtype == HB_BF16 && M >= 2048 && M % 1024 == 0)
                   ? (int)std::max<int64_t>(4, std::min<int64_t>(8, M / 1024)) : 1;
  if (chunks > 1) {
    const char* e = getenv("HB_HOST_CHUNKS");      // 4, 8 or 16: every one divides a multiple of 1024
    const int v = e ? atoi(e) : 0;
    if (v == 4 || v == 8 || v == 16) chunks = v;
  }
  if (chunks == 1) {
    if ((st = hb_upload(ctx, dA, A_host, a_b)) != HB_OK) return st;
    if ((st = hb_upload(ctx, dB, B_host, b_b)) != HB_OK) return st;
    hb_tensor tA = {dA, dtype, 2, {M, K, 0, 0}, {K, 1, 0, 0}};
    hb_tensor tB = {dB, dtype, 2, {K, N, 0, 0}, {1, K, 0, 0}};
    hb_tensor tC = {dC, dtype, 2, {M, N, 0, 0}, {N, 1, 0, 0}};
    if ((st = hb_matmul(ctx, &tA, &tB, &tC, nullptr)) != HB_OK) return st;
    if ((st = hb_download(ctx, C_host, dC, c_b)) != HB_OK) return st;
    return hb_sync(ctx);
  }
  cudaEvent_t* ev = nullptr;
  if ((st = hb_host_pipe(ctx, 2 * chunks + 2, &ev)) != HB_OK) return st;
  cudaEvent_t ev_start = ev[2 * chunks], ev_done = ev[2 * chunks + 1];
  const int64_t rows = M / chunks;
  HB_CUDA(ctx, cudaEventRecord(ev_start, ctx->stream));          // copies start after earlier work
  HB_CUDA(ctx, cudaStreamWaitEvent(ctx->h2d_stream, ev_start, 0));
  HB_CUDA(ctx, cudaStreamWaitEvent(ctx->d2h_stream, ev_start, 0));
  HB_CUDA(ctx, cudaMemcpyAsync(dB, B_host, b_b, cudaMemcpyHostToDevice, ctx->h2d_stream));
  for (int i = 0; i < chunks; ++i) {
    const size_t off = (size_t)i * rows * K * es;
    HB_CUDA(ctx, cudaMemcpyAsync(dA + off, static_cast<const char*>(A_host) + off, (size_t)rows * K * es,
                                 cudaMemcpyHostToDevice, ctx->h2d_stream));
    HB_CUDA(ctx, cudaEventRecord(ev[i], ctx->h2d_stream));
  }
  for (int i = 0; i < chunks; ++i) {
    HB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ev[i], 0));
    hb_tensor tA = {dA + (size_t)i * rows * K * es, dtype, 2, {rows, K, 0, 0}, {K, 1, 0, 0}};
    hb_tensor tB = {dB, dtype, 2, {K, N, 0, 0}, {1, K, 0, 0}};
    hb_tensor tC = {dC + (size_t)i * rows * N * es, dtype, 2, {rows, N, 0, 0}, {N, 1, 0, 0}};
    if ((st = hb_matmul(ctx, &tA, &tB, &tC, nullptr)) != HB_OK) return st;
    HB_CUDA(ctx, cudaEventRecord(ev[chunks + i], ctx->stream));
    HB_CUDA(ctx, cudaStreamWaitEvent(ctx->d2h_stream, ev[chunks + i], 0));
    const size_t coff = (size_t)i * rows * N * es;
    HB_CUDA(ctx, cudaMemcpyAsync(static_cast<char*>(C_host) + coff, dC + coff, (size_t)rows * N * es,
                                 cudaMemcpyDeviceToHost, ctx->d2h_stream));
  }
  HB_CUDA(ctx, cudaEventRecord(ev_done, ctx->d2h_stream));
  HB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ev_done, 0));
  return hb_sync(ctx);
}
