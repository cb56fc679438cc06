// fp32 GEMM on CUDA cores: C[M,N] = A[M,K] . B[K,N], fp32 storage; products are exact in
// double and are accumulated in double, so the only rounding is the final store (a
// single-pass TF32 tensor-core product, or fp32 accumulation where the sum cancels, would
// miss the 1e-4 relative tolerance this path is held to).  T x T output tile per CTA (64, or 32
// when 64-wide tiles would leave most SMs without one: the 256^3 case has 16 of them), 16 x 16
// threads, (T/16)^2 outputs per thread, 16-wide k-slices staged in shared memory.  Operands are
// addressed through (row stride, column stride) pairs, so row- and column-major inputs share
// one kernel.
#include "hb_internal.h"

namespace {

constexpr int TK = 16;

template <int T>
__global__ void __launch_bounds__(256)
hb_gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                   int M, int N, int K, int64_t a_rs, int64_t a_cs, int64_t b_rs, int64_t b_cs,
                   int64_t ldc) {
  __shared__ float sA[TK][T + 1];
  __shared__ float sB[TK][T + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * T, n0 = blockIdx.x * T;
  constexpr int R = T / 16;          // outputs per thread along each axis
  double acc[R][R] = {};
  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < T * TK; i += 256) {
      const int r = i / TK, kk = i % TK;   // A tile element (m0+r, k0+kk)
      const int gm = m0 + r, gk = k0 + kk;
      sA[kk][r] = (gm < M && gk < K) ? A[gm * a_rs + gk * a_cs] : 0.0f;
      const int gn = n0 + r;
      sB[kk][r] = (gn < N && gk < K) ? B[gk * b_rs + gn * b_cs] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[R], b[R];
#pragma unroll
      for (int i = 0; i < R; ++i) a[i] = sA[kk][ty * R + i];
#pragma unroll
      for (int j = 0; j < R; ++j) b[j] = sB[kk][tx * R + j];
#pragma unroll
      for (int i = 0; i < R; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) acc[i][j] = fma((double)a[i], (double)b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int gm = m0 + ty * R + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int gn = n0 + tx * R + j;
      if (gn < N) C[gm * ldc + gn] = (float)acc[i][j];
    }
  }
}

}  // namespace

hb_status hb_launch_gemm_f32(hb_ctx* ctx, const hb_gemm_args& a) {
  const int64_t a_rs = a.a_mn_major ? 1 : a.lda, a_cs = a.a_mn_major ? a.lda : 1;
  const int64_t b_rs = a.b_mn_major ? a.ldb : 1, b_cs = a.b_mn_major ? 1 : a.ldb;
  const bool small = ((a.N + 63) / 64) * ((a.M + 63) / 64) < ctx->sm_count;
  const int T = small ? 32 : 64;
  dim3 grid((unsigned)((a.N + T - 1) / T), (unsigned)((a.M + T - 1) / T));
  if (grid.y > 65535) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "matmul(f32): M too large");
  if (small)
    hb_gemm_f32_kernel<32><<<grid, 256, 0, ctx->stream>>>(
        static_cast<const float*>(a.A), static_cast<const float*>(a.B), static_cast<float*>(a.C),
        (int)a.M, (int)a.N, (int)a.K, a_rs, a_cs, b_rs, b_cs, a.ldc);
  else
    hb_gemm_f32_kernel<64><<<grid, 256, 0, ctx->stream>>>(
        static_cast<const float*>(a.A), static_cast<const float*>(a.B), static_cast<float*>(a.C),
        (int)a.M, (int)a.N, (int)a.K, a_rs, a_cs, b_rs, b_cs, a.ldc);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "gemm f32 launch");
}
