// HBM-bound glue operators of the decoder / MLP configurations: RMSNorm (+ fused residual
// add), rotate-half RoPE, embedding gather, SwiGLU, GELU (+ backward), add, argmax, MSE
// and Adam.  bf16 storage, fp32 math, 16-byte vector accesses; every kernel moves each
// byte once.
#include <math.h>

#include "hb_internal.h"

namespace {

__device__ __forceinline__ float2 bf2_to_f2(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
}
__device__ __forceinline__ uint32_t f2_to_bf2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------ RMSNorm
// One CTA per row, row held in registers (up to 8 x 16 B per thread).  Traffic per row:
// cols * 2 B in, cols * 2 B out (+ the same again for the residual stream when fused).
constexpr int RMS_THREADS = 256;
constexpr int RMS_MAX_VEC = 8;   // cols <= 256 * 8 * 8 = 16384

// Programmatic dependent launch (hb_launch_dependent): wait for the kernel in front before the
// first memory access, and let the kernel behind (e.g. the stream-K matmul, which streams its
// weights in before its own wait) start early.
#define HB_LAUNCH_DEPENDENTS() asm volatile("griddepcontrol.wait;\n\tgriddepcontrol.launch_dependents;" ::: "memory")

// VEC = 16-byte vectors per thread (cols <= 256 * 8 * VEC).  The row lives in registers, so the
// instantiation is chosen by the row length: a 4096-wide row needs 16 values per thread, not
// the 64 of the widest case, and four times as many CTAs fit on an SM (the kernel is bound by
// the bytes it has in flight).  The order of the arithmetic does not depend on VEC.
template <int VEC>
__global__ void __launch_bounds__(RMS_THREADS)
rmsnorm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ gain, uint4* __restrict__ y,
               uint4* residual, int cols8, float inv_cols, float eps) {
  __shared__ float red[RMS_THREADS / 32];
  HB_LAUNCH_DEPENDENTS();
  const int64_t row = blockIdx.x;
  const uint4* xr = x + row * cols8;
  uint4* rr = residual ? residual + row * cols8 : nullptr;
  float v[VEC][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = threadIdx.x + i * RMS_THREADS;
    if (c < cols8) {
      const uint4 a = xr[c];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
      uint32_t rw[4] = {0, 0, 0, 0};
      if (rr) { const uint4 r = rr[c]; rw[0] = r.x; rw[1] = r.y; rw[2] = r.z; rw[3] = r.w; }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 f = bf2_to_f2(aw[k]);
        if (rr) {
          const float2 g = bf2_to_f2(rw[k]);
          // the updated residual is what gets normalised, after its own bf16 rounding
          rw[k] = f2_to_bf2(f.x + g.x, f.y + g.y);
          f = bf2_to_f2(rw[k]);
        }
        v[i][2 * k] = f.x;
        v[i][2 * k + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
      if (rr) rr[c] = make_uint4(rw[0], rw[1], rw[2], rw[3]);
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < RMS_THREADS / 32; ++w) tot += red[w];
  const float inv = rsqrtf(tot * inv_cols + eps);
  uint4* yr = y + row * cols8;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = threadIdx.x + i * RMS_THREADS;
    if (c < cols8) {
      const uint4 g = __ldg(gain + c);
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 gf = bf2_to_f2(gw[k]);
        o[k] = f2_to_bf2(v[i][2 * k] * inv * gf.x, v[i][2 * k + 1] * inv * gf.y);
      }
      yr[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ------------------------------------------------------------------ RoPE (rotate-half)
// cos/sin of pos * base^(-2i/d) are tabulated once per (seq, head_dim, base, pos0): the
// angle is formed in double and reduced by sincos in double, so the table carries no
// large-angle error.  table[p * half + i] = (cos, sin).
__global__ void rope_table_kernel(float2* table, int seq, int half, int head_dim, double log2_base, int64_t pos0) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= seq * half) return;
  const int i = idx % half;
  const double pos = (double)(pos0 + idx / half);
  const double th = pos * exp2(-2.0 * i / head_dim * log2_base);
  double s, c;
  sincos(th, &s, &c);
  table[idx] = make_float2((float)c, (float)s);
}

// One thread per (token, head, 8 consecutive pair indices): 16 B from each half of the
// head and 64 B of table.  Traffic: the rotated slice once in, once out.
__global__ void rope_kernel(__nv_bfloat16* x, const float2* __restrict__ table, int64_t tokens, int seq, int heads,
                            int head_dim, int64_t row_stride) {
  const int half = head_dim >> 1;
  const int groups = half >> 3;
  const int64_t total = tokens * heads * groups;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int g = (int)(idx % groups);
    const int h = (int)((idx / groups) % heads);
    const int64_t t = idx / ((int64_t)groups * heads);
    const float4* cs = reinterpret_cast<const float4*>(table + (t % seq) * half + g * 8);
    __nv_bfloat16* base = x + t * row_stride + (int64_t)h * head_dim + g * 8;
    uint4 lo = *reinterpret_cast<uint4*>(base);
    uint4 hi = *reinterpret_cast<uint4*>(base + half);
    uint32_t* lw = reinterpret_cast<uint32_t*>(&lo);
    uint32_t* hw = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = bf2_to_f2(lw[k]);
      const float2 b = bf2_to_f2(hw[k]);
      const float4 t4 = __ldg(cs + k);           // (c0, s0, c1, s1)
      lw[k] = f2_to_bf2(a.x * t4.x - b.x * t4.y, a.y * t4.z - b.y * t4.w);
      hw[k] = f2_to_bf2(b.x * t4.x + a.x * t4.y, b.y * t4.z + a.y * t4.w);
    }
    *reinterpret_cast<uint4*>(base) = lo;
    *reinterpret_cast<uint4*>(base + half) = hi;
  }
}

// ------------------------------------------------------------------ embedding gather
__global__ void embedding_kernel(const uint4* __restrict__ table, const int32_t* __restrict__ ids,
                                 uint4* __restrict__ out, int64_t tokens, int vocab, int dim8,
                                 int32_t* status) {
  const int64_t total = tokens * dim8;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / dim8;
    const int c = (int)(idx % dim8);
    const int id = ids[t];
    if (id < 0 || id >= vocab) {   // record and skip: never read out of bounds
      if (c == 0) { atomicCAS(status, 0, HB_ERR_INVALID); status[1] = 10; status[2] = id; }
      out[idx] = make_uint4(0, 0, 0, 0);
      continue;
    }
    out[idx] = table[(int64_t)id * dim8 + c];
  }
}

// ------------------------------------------------------------------ elementwise
__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + __expf(-v)); }
__device__ __forceinline__ float gelu_f(float v) { return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f)); }

// out[r, j] = silu(x[r, j]) * x[r, half + j]; half8 = half / 8
__global__ void swiglu_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, int64_t rows, int half8) {
  HB_LAUNCH_DEPENDENTS();
  const int64_t total = rows * half8;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / half8;
    const int c = (int)(idx % half8);
    const uint4 g = x[r * 2 * half8 + c], u = x[r * 2 * half8 + half8 + c];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = bf2_to_f2(gw[k]), b = bf2_to_f2(uw[k]);
      o[k] = f2_to_bf2(silu_f(a.x) * b.x, silu_f(a.y) * b.y);
    }
    out[idx] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <int OP>  // 0 gelu(x), 1 a + b, 2 gelu'(a) * b
__global__ void ew_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out,
                          int64_t n8, const __nv_bfloat16* at, const __nv_bfloat16* bt, __nv_bfloat16* ot,
                          int tail) {
  HB_LAUNCH_DEPENDENTS();
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < n8;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const uint4 av = a[idx];
    uint4 bv = make_uint4(0, 0, 0, 0);
    if (OP != 0) bv = b[idx];
    const uint32_t aw[4] = {av.x, av.y, av.z, av.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = bf2_to_f2(aw[k]), y = bf2_to_f2(bw[k]);
      if (OP == 0) o[k] = f2_to_bf2(gelu_f(x.x), gelu_f(x.y));
      else if (OP == 1) o[k] = f2_to_bf2(x.x + y.x, x.y + y.y);
      else {
        auto dg = [](float v) {
          return 0.5f * (1.0f + erff(v * 0.70710678118654752f)) + v * 0.3989422804014327f * __expf(-0.5f * v * v);
        };
        o[k] = f2_to_bf2(dg(x.x) * y.x, dg(x.y) * y.y);
      }
    }
    out[idx] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (blockIdx.x == 0 && threadIdx.x < tail) {   // last n % 8 elements
    const float x = __bfloat162float(at[threadIdx.x]);
    const float y = OP != 0 ? __bfloat162float(bt[threadIdx.x]) : 0.f;
    float r;
    if (OP == 0) r = gelu_f(x);
    else if (OP == 1) r = x + y;
    else r = (0.5f * (1.0f + erff(x * 0.70710678118654752f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x)) * y;
    ot[threadIdx.x] = __float2bfloat16_rn(r);
  }
}

// ------------------------------------------------------------------ argmax (first index wins)
__global__ void __launch_bounds__(256)
argmax_kernel(const __nv_bfloat16* __restrict__ x, int32_t* __restrict__ out, int64_t cols) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const __nv_bfloat16* xr = x + blockIdx.x * cols;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int64_t c = threadIdx.x; c < cols; c += 256) {
    const float v = __bfloat162float(xr[c]);
    if (v > bv || (v == bv && (int)c < bi)) { bv = v; bi = (int)c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
    out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

int grid_for(hb_ctx* ctx, int64_t work_items, int threads) {
  const int64_t want = (work_items + threads - 1) / threads;
  const int64_t cap = (int64_t)ctx->sm_count * 8;   // a multiple of the SM count
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace

#define HB_ALIGNED16(p) ((reinterpret_cast<uintptr_t>(p) & 15) == 0)

extern "C" hb_status hb_rmsnorm(hb_ctx* ctx, const void* x, const void* gain, void* y, void* residual_inout,
                                int64_t rows, int64_t cols, float eps) {
  if (!ctx) return HB_ERR_INVALID;
  if (!x || !gain || !y) return hb_fail(ctx, HB_ERR_INVALID, "rmsnorm: null pointer");
  if (rows <= 0 || cols <= 0) return hb_fail(ctx, HB_ERR_INVALID, "rmsnorm: empty dimension");
  if (cols % 8 || cols > RMS_THREADS * RMS_MAX_VEC * 8)
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "rmsnorm: cols must be a multiple of 8 and at most %d",
                   RMS_THREADS * RMS_MAX_VEC * 8);
  if (!HB_ALIGNED16(x) || !HB_ALIGNED16(gain) || !HB_ALIGNED16(y) || !HB_ALIGNED16(residual_inout))
    return hb_fail(ctx, HB_ERR_INVALID, "rmsnorm: pointers must be 16-byte aligned");
  if (rows > INT32_MAX) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "rmsnorm: too many rows");
  const int vec = (int)((cols / 8 + RMS_THREADS - 1) / RMS_THREADS);
#define HB_RMS_LAUNCH(V)                                                                                  \
  hb_launch_dependent(rmsnorm_kernel<V>, dim3((unsigned)rows), dim3(RMS_THREADS), 0, ctx->stream,       \
                      static_cast<const uint4*>(x), static_cast<const uint4*>(gain), static_cast<uint4*>(y), \
                      static_cast<uint4*>(residual_inout), (int)(cols / 8), 1.0f / (float)cols, eps)
  if (vec <= 1) HB_RMS_LAUNCH(1);
  else if (vec <= 2) HB_RMS_LAUNCH(2);
  else if (vec <= 4) HB_RMS_LAUNCH(4);
  else HB_RMS_LAUNCH(RMS_MAX_VEC);
#undef HB_RMS_LAUNCH
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "rmsnorm launch");
}

extern "C" hb_status hb_rope(hb_ctx* ctx, void* x, int64_t tokens, int64_t seq, int64_t heads, int64_t head_dim,
                             int64_t row_stride, float base, int64_t pos0) {
  if (!ctx) return HB_ERR_INVALID;
  if (!x) return hb_fail(ctx, HB_ERR_INVALID, "rope: null pointer");
  if (tokens <= 0 || seq <= 0 || heads <= 0 || head_dim <= 0) return hb_fail(ctx, HB_ERR_INVALID, "rope: empty dimension");
  if (head_dim % 16 || row_stride % 8 || !HB_ALIGNED16(x))
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "rope: head_dim must be a multiple of 16 and rows 16-byte aligned");
  if (row_stride < heads * head_dim) return hb_fail(ctx, HB_ERR_INVALID, "rope: row stride smaller than heads * head_dim");
  if (!(base > 1.0f)) return hb_fail(ctx, HB_ERR_INVALID, "rope: base must exceed 1");
  if (seq > (1 << 22)) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "rope: sequence too long");
  const int half = (int)head_dim / 2;
  if (!ctx->rope_table || ctx->rope_seq != seq || ctx->rope_head_dim != head_dim || ctx->rope_base != base ||
      ctx->rope_pos0 != pos0) {
    const size_t bytes = (size_t)seq * half * sizeof(float2);
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaSetDevice");
    if (bytes > ctx->rope_table_bytes) {
      if (ctx->rope_table) { hb_quiesce(ctx); cudaFree(ctx->rope_table); ctx->rope_table = nullptr; }
      e = cudaMalloc(&ctx->rope_table, bytes);
      if (e != cudaSuccess) { cudaGetLastError(); ctx->rope_table_bytes = 0; return hb_fail(ctx, HB_ERR_NOMEM, "rope: cannot allocate the angle table"); }
      ctx->rope_table_bytes = bytes;
    }
    rope_table_kernel<<<(unsigned)((seq * half + 255) / 256), 256, 0, ctx->stream>>>(
        static_cast<float2*>(ctx->rope_table), (int)seq, half, (int)head_dim, log2((double)base), pos0);
    ctx->launches++;
    ctx->rope_seq = seq; ctx->rope_head_dim = head_dim; ctx->rope_base = base; ctx->rope_pos0 = pos0;
  }
  const int64_t work = tokens * heads * (head_dim / 16);
  rope_kernel<<<grid_for(ctx, work, 256), 256, 0, ctx->stream>>>(static_cast<__nv_bfloat16*>(x),
                                                                 static_cast<const float2*>(ctx->rope_table), tokens,
                                                                 (int)seq, (int)heads, (int)head_dim, row_stride);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "rope launch");
}

extern "C" hb_status hb_embedding(hb_ctx* ctx, const void* table, const int32_t* ids, void* out, int64_t tokens,
                                  int64_t vocab, int64_t dim) {
  if (!ctx) return HB_ERR_INVALID;
  if (!table || !ids || !out) return hb_fail(ctx, HB_ERR_INVALID, "embedding: null pointer");
  if (tokens <= 0 || vocab <= 0 || dim <= 0) return hb_fail(ctx, HB_ERR_INVALID, "embedding: empty dimension");
  if (dim % 8 || !HB_ALIGNED16(table) || !HB_ALIGNED16(out) || vocab > INT32_MAX)
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "embedding: dim must be a multiple of 8 and pointers 16-byte aligned");
  embedding_kernel<<<grid_for(ctx, tokens * (dim / 8), 256), 256, 0, ctx->stream>>>(
      static_cast<const uint4*>(table), ids, static_cast<uint4*>(out), tokens, (int)vocab, (int)(dim / 8),
      ctx->d_status);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "embedding launch");
}

extern "C" hb_status hb_swiglu(hb_ctx* ctx, const void* x, void* out, int64_t rows, int64_t half) {
  if (!ctx) return HB_ERR_INVALID;
  if (!x || !out) return hb_fail(ctx, HB_ERR_INVALID, "swiglu: null pointer");
  if (rows <= 0 || half <= 0) return hb_fail(ctx, HB_ERR_INVALID, "swiglu: empty dimension");
  if (half % 8 || !HB_ALIGNED16(x) || !HB_ALIGNED16(out))
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "swiglu: half width must be a multiple of 8 and pointers 16-byte aligned");
  hb_launch_dependent(swiglu_kernel, dim3(grid_for(ctx, rows * (half / 8), 256)), dim3(256), 0, ctx->stream,
      static_cast<const uint4*>(x), static_cast<uint4*>(out), rows, (int)(half / 8));
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "swiglu launch");
}

template <int OP>
static hb_status launch_ew(hb_ctx* ctx, const char* name, const void* a, const void* b, void* out, int64_t n) {
  if (!ctx) return HB_ERR_INVALID;
  if (!a || !out || (OP != 0 && !b)) return hb_fail(ctx, HB_ERR_INVALID, "%s: null pointer", name);
  if (n <= 0) return hb_fail(ctx, HB_ERR_INVALID, "%s: empty tensor", name);
  if (!HB_ALIGNED16(a) || !HB_ALIGNED16(b) || !HB_ALIGNED16(out))
    return hb_fail(ctx, HB_ERR_INVALID, "%s: pointers must be 16-byte aligned", name);
  const int64_t n8 = n / 8;
  const int tail = (int)(n % 8);
  const __nv_bfloat16* at = static_cast<const __nv_bfloat16*>(a) + n8 * 8;
  const __nv_bfloat16* bt = b ? static_cast<const __nv_bfloat16*>(b) + n8 * 8 : nullptr;
  __nv_bfloat16* ot = static_cast<__nv_bfloat16*>(out) + n8 * 8;
  hb_launch_dependent(ew_kernel<OP>, dim3(grid_for(ctx, n8, 256)), dim3(256), 0, ctx->stream,
      static_cast<const uint4*>(a), static_cast<const uint4*>(b), static_cast<uint4*>(out), n8, at, bt, ot, tail);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), name);
}

extern "C" hb_status hb_gelu(hb_ctx* ctx, const void* x, void* y, int64_t n) {
  return launch_ew<0>(ctx, "gelu", x, nullptr, y, n);
}
extern "C" hb_status hb_add(hb_ctx* ctx, const void* a, const void* b, void* out, int64_t n) {
  return launch_ew<1>(ctx, "add", a, b, out, n);
}
extern "C" hb_status hb_gelu_backward(hb_ctx* ctx, const void* x, const void* dy, void* dx, int64_t n) {
  return launch_ew<2>(ctx, "gelu_backward", x, dy, dx, n);
}

extern "C" hb_status hb_argmax(hb_ctx* ctx, const void* x, int32_t* out, int64_t rows, int64_t cols) {
  if (!ctx) return HB_ERR_INVALID;
  if (!x || !out) return hb_fail(ctx, HB_ERR_INVALID, "argmax: null pointer");
  if (rows <= 0 || cols <= 0 || rows > INT32_MAX || cols > INT32_MAX)
    return hb_fail(ctx, HB_ERR_INVALID, "argmax: bad dimensions");
  argmax_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(static_cast<const __nv_bfloat16*>(x), out, cols);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "argmax launch");
}

// ------------------------------------------------------------------ MSE loss and Adam
namespace {

// dY = 2 (y - t) / n (bf16), per-block partial sums of (y - t)^2 in fixed slots.
__global__ void __launch_bounds__(256)
mse_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ t, __nv_bfloat16* __restrict__ dy,
           float* __restrict__ partial, int64_t n, float two_over_n) {
  __shared__ float red[8];
  float s = 0.f;
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    const float d = __bfloat162float(y[i]) - __bfloat162float(t[i]);
    s += d * d;
    dy[i] = __float2bfloat16_rn(d * two_over_n);
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < 8; ++w) tot += red[w];
    partial[blockIdx.x] = tot;
  }
}
// loss = sum(partial[0..m)) / n, added in index order by one warp (deterministic).
__global__ void mse_finish_kernel(const float* __restrict__ partial, int m, float inv_n, float* __restrict__ loss) {
  double s = 0.0;
  for (int i = threadIdx.x; i < m; i += 32) s += (double)partial[i];
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (threadIdx.x == 0) *loss = (float)(s * (double)inv_n);
}

// Bias-corrected Adam on fp32 master weights and moments; the gradient arrives in bf16
// (scaled by grad_scale, e.g. 1/world after a sum-allreduce) and the bf16 compute copy of
// the weights is refreshed in the same pass: 2 + 12 bytes read, 12 + 2 written per weight.
__global__ void __launch_bounds__(256)
adam_kernel(float4* __restrict__ w, float4* __restrict__ m, float4* __restrict__ v, const uint2* __restrict__ g,
            uint2* __restrict__ wb, int64_t n4, float lr, float b1, float b2, float eps, float c1, float c2,
            float grad_scale) {
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < n4; i += (int64_t)gridDim.x * 256) {
    const uint2 gr = g[i];
    const float2 g01 = bf2_to_f2(gr.x), g23 = bf2_to_f2(gr.y);
    const float gv[4] = {g01.x * grad_scale, g01.y * grad_scale, g23.x * grad_scale, g23.y * grad_scale};
    float4 wv = w[i], mv = m[i], vv = v[i];
    float* wp = reinterpret_cast<float*>(&wv);
    float* mp = reinterpret_cast<float*>(&mv);
    float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mp[k] = b1 * mp[k] + (1.0f - b1) * gv[k];
      vp[k] = b2 * vp[k] + (1.0f - b2) * gv[k] * gv[k];
      const float mh = mp[k] / c1, vh = vp[k] / c2;
      wp[k] = wp[k] - lr * mh / (sqrtf(vh) + eps);
    }
    w[i] = wv; m[i] = mv; v[i] = vv;
    wb[i] = make_uint2(f2_to_bf2(wp[0], wp[1]), f2_to_bf2(wp[2], wp[3]));
  }
}

}  // namespace

extern "C" hb_status hb_mse(hb_ctx* ctx, const void* y, const void* target, void* dy, float* loss, int64_t n) {
  if (!ctx) return HB_ERR_INVALID;
  if (!y || !target || !dy || !loss) return hb_fail(ctx, HB_ERR_INVALID, "mse: null pointer");
  if (n <= 0) return hb_fail(ctx, HB_ERR_INVALID, "mse: empty tensor");
  const int grid = grid_for(ctx, n, 256);
  void* ws = nullptr;
  hb_status st = hb_get_scratch(ctx, HB_SCRATCH_REDUCE, (size_t)grid * sizeof(float), &ws);
  if (st != HB_OK) return st;
  mse_kernel<<<grid, 256, 0, ctx->stream>>>(static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(target),
                                            static_cast<__nv_bfloat16*>(dy), static_cast<float*>(ws), n, 2.0f / (float)n);
  mse_finish_kernel<<<1, 32, 0, ctx->stream>>>(static_cast<const float*>(ws), grid, 1.0f / (float)n, loss);
  ctx->launches += 2;
  return hb_check_cuda(ctx, cudaGetLastError(), "mse launch");
}

extern "C" hb_status hb_adam_step(hb_ctx* ctx, float* w, float* m, float* v, const void* grad_bf16, void* w_bf16,
                                  int64_t n, float lr, float beta1, float beta2, float eps, int64_t step,
                                  float grad_scale) {
  if (!ctx) return HB_ERR_INVALID;
  if (!w || !m || !v || !grad_bf16 || !w_bf16) return hb_fail(ctx, HB_ERR_INVALID, "adam: null pointer");
  if (n <= 0 || n % 4) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "adam: element count must be a positive multiple of 4");
  if (step < 1) return hb_fail(ctx, HB_ERR_INVALID, "adam: step counts from 1");
  if (!HB_ALIGNED16(w) || !HB_ALIGNED16(m) || !HB_ALIGNED16(v) || (reinterpret_cast<uintptr_t>(grad_bf16) & 7) ||
      (reinterpret_cast<uintptr_t>(w_bf16) & 7))
    return hb_fail(ctx, HB_ERR_INVALID, "adam: misaligned pointer");
  const float c1 = (float)(1.0 - pow((double)beta1, (double)step));
  const float c2 = (float)(1.0 - pow((double)beta2, (double)step));
  // The update may run on the side stream beside the backward products (hb_adam_step_async): it
  // then shares SMs with GEMM CTAs, which only works under the GEMM's L1 / shared-memory split.
  static bool carve_set[64] = {};
  if (!carve_set[ctx->device & 63]) {
    cudaFuncSetAttribute(adam_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaGetLastError();
    carve_set[ctx->device & 63] = true;
  }
  adam_kernel<<<grid_for(ctx, n / 4, 256), 256, 0, ctx->stream>>>(
      reinterpret_cast<float4*>(w), reinterpret_cast<float4*>(m), reinterpret_cast<float4*>(v),
      static_cast<const uint2*>(grad_bf16), static_cast<uint2*>(w_bf16), n / 4, lr, beta1, beta2, eps, c1, c2, grad_scale);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "adam launch");
}

// The same update on the context's high-priority side stream, ordered after everything queued on
// the main stream so far (like hb_all_reduce_async; hb_side_join makes the main stream wait).
// The optimizer step is bound by HBM (30 bytes per weight) and the backward products by the
// tensor cores, so the update of a layer whose gradient is complete runs under the products of
// the layers still to come.  Kernels queued on the main stream between this call and
// hb_side_join must not touch the layer's weights, moments or gradient.
extern "C" hb_status hb_adam_step_async(hb_ctx* ctx, float* w, float* m, float* v, const void* grad_bf16, void* w_bf16,
                                        int64_t n, float lr, float beta1, float beta2, float eps, int64_t step,
                                        float grad_scale) {
  if (!ctx) return HB_ERR_INVALID;
  if (!ctx->side_stream) {
    int lo = 0, hi = 0;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);
    cudaError_t e = cudaStreamCreateWithPriority(&ctx->side_stream, cudaStreamNonBlocking, hi);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaStreamCreate(side)");
  }
  if (!ctx->side_event) {
    cudaError_t e = cudaEventCreateWithFlags(&ctx->side_event, cudaEventDisableTiming);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaEventCreate(side)");
  }
  cudaStream_t main_stream = ctx->stream;
  cudaError_t e = cudaEventRecord(ctx->side_event, main_stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->side_stream, ctx->side_event, 0);
  if (e != cudaSuccess) return hb_check_cuda(ctx, e, "adam_step_async: fork");
  ctx->stream = ctx->side_stream;
  const hb_status st = hb_adam_step(ctx, w, m, v, grad_bf16, w_bf16, n, lr, beta1, beta2, eps, step, grad_scale);
  ctx->stream = main_stream;
  return st;
}
