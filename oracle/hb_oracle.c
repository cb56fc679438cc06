/*
 * hb_oracle.c -- CPU restatement of the dense hot path, used ONLY as the checker for the
 * CUDA library (tests, the smoke check and the bench's CPU-baseline leg).  It is test
 * infrastructure: nothing in the product path calls it.
 *
 * PARITY UNPINNED.  The reference project (joelreymont/habu) contains no implementation
 * of this path -- no matmul, attention, collective, executor or any numeric code; its
 * `MUL` / `FMUL` (`src/lib/sleigh.ml:219,224`) are syntax constructors that nothing
 * evaluates, and its 24 tests (`test/sleigh_parser_test.ml:13-231`) pin only printed
 * parse trees.  There is therefore no reference file to follow and no golden vector to
 * pin against; the functions below restate the textbook definitions at the shapes,
 * dtypes and constants the benchmark configurations name:
 *   GEMM          C = A.B, fp32 (or double) accumulation
 *   attention     O = softmax(scale * Q K^T + causal mask) V, fp32 row max / sum
 *   RMSNorm       y = x * rsqrt(mean(x^2) + eps) * g
 *   RoPE          rotate-half pairing (i, i + d/2), theta_i = base^(-2i/d)
 *   SwiGLU        silu(gate) * up;  GELU erf-exact;  MSE mean over all elements
 *   Adam          bias-corrected, no weight decay
 * All tensors are fp32 in memory; "bf16" inputs are fp32 values already rounded to bf16
 * (round-to-nearest-even) by orc_round_bf16, so the device consumes the same numbers.
 *
 * Build: make -C oracle   (gcc -O3 -fopenmp, x86-64-v3 so the .so runs on any AVX2 host)
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ bf16 helpers */
static inline uint16_t f32_to_bf16_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* quiet NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb; /* round to nearest, ties to even */
  return (uint16_t)(u >> 16);
}
static inline float bf16_bits_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
void orc_f32_to_bf16(const float* x, uint16_t* y, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) y[i] = f32_to_bf16_bits(x[i]);
}
void orc_bf16_to_f32(const uint16_t* x, float* y, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) y[i] = bf16_bits_to_f32(x[i]);
}
void orc_round_bf16(float* x, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) x[i] = bf16_bits_to_f32(f32_to_bf16_bits(x[i]));
}

/* ------------------------------------------------------------------ seeded inputs
 * Counter-based: element i of stream `seed` depends only on (seed, i), so any rank can
 * generate its own shard.  SplitMix64 finaliser over seed * golden + i. */
static inline uint64_t mix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}
static inline double u01(uint64_t seed, uint64_t i) { /* (0,1) */
  uint64_t r = mix64(mix64(seed) ^ (i * 0xd1342543de82ef95ull));
  return ((double)(r >> 11) + 0.5) * (1.0 / 9007199254740992.0);
}
void orc_fill_uniform(float* x, int64_t n, uint64_t seed, int64_t offset, float lo, float hi) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) x[i] = (float)(lo + (hi - lo) * u01(seed, (uint64_t)(offset + i)));
}
void orc_fill_normal(float* x, int64_t n, uint64_t seed, int64_t offset, float mean, float std) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) { /* Box-Muller, one normal per index */
    const uint64_t j = (uint64_t)(offset + i);
    const double u1 = u01(seed, 2 * j), u2 = u01(seed, 2 * j + 1);
    x[i] = (float)(mean + std * sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2));
  }
}

/* ------------------------------------------------------------------ GEMM
 * C[m,n] = sum_k A[m,k] * B[k,n].  A addressed as A[m*a_rs + k*a_cs], B as
 * B[k*b_rs + n*b_cs].  acc_double != 0 accumulates in double (strict reference for the
 * fp32 path); otherwise fp32 accumulation in 16-wide partial sums. */
static float* pack_kmajor(const float* X, int64_t R, int64_t K, int64_t rs, int64_t cs) {
  if (cs == 1 && rs == K) return NULL; /* already K-contiguous and dense */
  float* P = (float*)malloc((size_t)R * K * sizeof(float));
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < R; ++r)
    for (int64_t k = 0; k < K; ++k) P[r * K + k] = X[r * rs + k * cs];
  return P;
}
void orc_gemm(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
              int64_t a_rs, int64_t a_cs, int64_t b_rs, int64_t b_cs, int64_t ldc,
              int acc_double) {
  float* Ap = pack_kmajor(A, M, K, a_rs, a_cs);
  float* Bp = pack_kmajor(B, N, K, b_cs, b_rs); /* rows of Bp are columns of B */
  const float* a = Ap ? Ap : A;
  const float* b = Bp ? Bp : B;
  if (acc_double) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m)
      for (int64_t n = 0; n < N; ++n) {
        double s = 0.0;
        const float* ar = a + m * K;
        const float* br = b + n * K;
        for (int64_t k = 0; k < K; ++k) s += (double)ar[k] * (double)br[k];
        C[m * ldc + n] = (float)s;
      }
  } else {
    enum { TM = 4, TN = 4, KB = 1024 };
    const int64_t mb = (M + TM - 1) / TM;
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t bi = 0; bi < mb; ++bi) {
      const int64_t m0 = bi * TM, mh = (m0 + TM <= M) ? TM : (M - m0);
      for (int64_t n0 = 0; n0 < N; n0 += TN) {
        const int64_t nh = (n0 + TN <= N) ? TN : (N - n0);
        float acc[TM][TN];
        for (int i = 0; i < TM; ++i)
          for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
        if (mh == TM && nh == TN) {
          for (int64_t k0 = 0; k0 < K; k0 += KB) {
            const int64_t k1 = k0 + KB < K ? k0 + KB : K;
            float s00 = 0, s01 = 0, s02 = 0, s03 = 0, s10 = 0, s11 = 0, s12 = 0, s13 = 0;
            float s20 = 0, s21 = 0, s22 = 0, s23 = 0, s30 = 0, s31 = 0, s32 = 0, s33 = 0;
            const float *a0 = a + (m0 + 0) * K, *a1 = a + (m0 + 1) * K, *a2 = a + (m0 + 2) * K,
                        *a3 = a + (m0 + 3) * K;
            const float *b0 = b + (n0 + 0) * K, *b1 = b + (n0 + 1) * K, *b2 = b + (n0 + 2) * K,
                        *b3 = b + (n0 + 3) * K;
#pragma omp simd reduction(+ : s00, s01, s02, s03, s10, s11, s12, s13, s20, s21, s22, s23, s30, s31, s32, s33)
            for (int64_t k = k0; k < k1; ++k) {
              s00 += a0[k] * b0[k]; s01 += a0[k] * b1[k]; s02 += a0[k] * b2[k]; s03 += a0[k] * b3[k];
              s10 += a1[k] * b0[k]; s11 += a1[k] * b1[k]; s12 += a1[k] * b2[k]; s13 += a1[k] * b3[k];
              s20 += a2[k] * b0[k]; s21 += a2[k] * b1[k]; s22 += a2[k] * b2[k]; s23 += a2[k] * b3[k];
              s30 += a3[k] * b0[k]; s31 += a3[k] * b1[k]; s32 += a3[k] * b2[k]; s33 += a3[k] * b3[k];
            }
            acc[0][0] += s00; acc[0][1] += s01; acc[0][2] += s02; acc[0][3] += s03;
            acc[1][0] += s10; acc[1][1] += s11; acc[1][2] += s12; acc[1][3] += s13;
            acc[2][0] += s20; acc[2][1] += s21; acc[2][2] += s22; acc[2][3] += s23;
            acc[3][0] += s30; acc[3][1] += s31; acc[3][2] += s32; acc[3][3] += s33;
          }
        } else {
          for (int64_t i = 0; i < mh; ++i)
            for (int64_t j = 0; j < nh; ++j) {
              float s = 0.f;
              const float* ar = a + (m0 + i) * K;
              const float* br = b + (n0 + j) * K;
#pragma omp simd reduction(+ : s)
              for (int64_t k = 0; k < K; ++k) s += ar[k] * br[k];
              acc[i][j] = s;
            }
        }
        for (int64_t i = 0; i < mh; ++i)
          for (int64_t j = 0; j < nh; ++j) C[(m0 + i) * ldc + n0 + j] = acc[i][j];
      }
    }
  }
  free(Ap);
  free(Bp);
}

/* ------------------------------------------------------------------ attention
 * Q [B,S,Hq,D], K/V [B,S,Hkv,D], O [B,S,Hq,D] (token-major), Hq % Hkv == 0; query head h
 * reads KV head h / (Hq/Hkv).  fp32 scores, fp32 max/sum.  round_p != 0 rounds the
 * un-normalised probabilities exp(s - max) to bf16 before the PV product, as the device
 * does; the row sum is taken of the unrounded values.  lse (optional) [B,Hq,S]. */
void orc_attention(const float* Q, const float* K, const float* V, float* O, float* lse,
                   int64_t B, int64_t S, int64_t Hq, int64_t Hkv, int64_t D, int causal,
                   float scale, int round_p) {
  const int64_t grp = Hq / Hkv;
#pragma omp parallel
  {
    float* p = (float*)malloc((size_t)S * sizeof(float));
    double* o = (double*)malloc((size_t)D * sizeof(double));
#pragma omp for collapse(3) schedule(dynamic, 8)
    for (int64_t b = 0; b < B; ++b)
      for (int64_t h = 0; h < Hq; ++h)
        for (int64_t i = 0; i < S; ++i) {
          const int64_t hk = h / grp;
          const float* q = Q + ((b * S + i) * Hq + h) * D;
          const int64_t jn = causal ? i + 1 : S;
          float mx = -INFINITY;
          for (int64_t j = 0; j < jn; ++j) {
            const float* k = K + ((b * S + j) * Hkv + hk) * D;
            float s = 0.f;
#pragma omp simd reduction(+ : s)
            for (int64_t d = 0; d < D; ++d) s += q[d] * k[d];
            s *= scale;
            p[j] = s;
            if (s > mx) mx = s;
          }
          double sum = 0.0;
          for (int64_t j = 0; j < jn; ++j) {
            const float e = expf(p[j] - mx);
            sum += e;
            p[j] = round_p ? bf16_bits_to_f32(f32_to_bf16_bits(e)) : e;
          }
          for (int64_t d = 0; d < D; ++d) o[d] = 0.0;
          for (int64_t j = 0; j < jn; ++j) {
            const float* v = V + ((b * S + j) * Hkv + hk) * D;
            const double pj = p[j];
            for (int64_t d = 0; d < D; ++d) o[d] += pj * v[d];
          }
          float* out = O + ((b * S + i) * Hq + h) * D;
          for (int64_t d = 0; d < D; ++d) out[d] = (float)(o[d] / sum);
          if (lse) lse[(b * Hq + h) * S + i] = mx + (float)log(sum);
        }
    free(p);
    free(o);
  }
}

/* ------------------------------------------------------------------ glue */
void orc_rmsnorm(const float* x, const float* gain, float* y, int64_t rows, int64_t cols,
                 float eps) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    double ss = 0.0;
    for (int64_t c = 0; c < cols; ++c) ss += (double)xr[c] * xr[c];
    const float inv = (float)(1.0 / sqrt(ss / (double)cols + (double)eps));
    for (int64_t c = 0; c < cols; ++c) y[r * cols + c] = xr[c] * inv * gain[c];
  }
}
/* In place over x[tokens, heads, head_dim] with row pitch row_stride (elements);
 * token t sits at position pos0 + t % seq; pairs (i, i + head_dim/2). */
void orc_rope(float* x, int64_t tokens, int64_t seq, int64_t heads, int64_t head_dim,
              int64_t row_stride, float base, int64_t pos0) {
  const int64_t half = head_dim / 2;
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < tokens; ++t) {
    const double pos = (double)(pos0 + t % seq);
    for (int64_t h = 0; h < heads; ++h) {
      float* v = x + t * row_stride + h * head_dim;
      for (int64_t i = 0; i < half; ++i) {
        const double theta = pos * pow((double)base, -2.0 * (double)i / (double)head_dim);
        const float c = (float)cos(theta), s = (float)sin(theta);
        const float a = v[i], b = v[i + half];
        v[i] = a * c - b * s;
        v[i + half] = b * c + a * s;
      }
    }
  }
}
static inline float silu_f(float x) { return x / (1.0f + expf(-x)); }
static inline float gelu_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }
/* out[r,j] = silu(x[r,j]) * x[r, half+j] */
void orc_swiglu(const float* x, float* out, int64_t rows, int64_t half) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t j = 0; j < half; ++j)
      out[r * half + j] = silu_f(x[r * 2 * half + j]) * x[r * 2 * half + half + j];
}
/* interleaved variant: out[r,j] = silu(x[r,2j]) * x[r,2j+1] */
void orc_swiglu_interleaved(const float* x, float* out, int64_t rows, int64_t half) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t j = 0; j < half; ++j)
      out[r * half + j] = silu_f(x[r * 2 * half + 2 * j]) * x[r * 2 * half + 2 * j + 1];
}
void orc_gelu(const float* x, float* y, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) y[i] = gelu_f(x[i]);
}
/* dx = dy * gelu'(x), erf-exact */
void orc_gelu_backward(const float* x, const float* dy, float* dx, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float v = x[i];
    const float cdf = 0.5f * (1.0f + erff(v * 0.70710678118654752f));
    const float pdf = 0.3989422804014327f * expf(-0.5f * v * v);
    dx[i] = dy[i] * (cdf + v * pdf);
  }
}
void orc_add(const float* a, const float* b, float* out, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}
void orc_embedding(const float* table, const int32_t* ids, float* out, int64_t tokens,
                   int64_t dim) {
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < tokens; ++t)
    memcpy(out + t * dim, table + (int64_t)ids[t] * dim, (size_t)dim * sizeof(float));
}
/* first maximal index per row */
void orc_argmax(const float* x, int32_t* out, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    int32_t best = 0;
    float bv = x[r * cols];
    for (int64_t c = 1; c < cols; ++c)
      if (x[r * cols + c] > bv) { bv = x[r * cols + c]; best = (int32_t)c; }
    out[r] = best;
  }
}
double orc_mse(const float* y, const float* t, int64_t n) {
  double s = 0.0;
#pragma omp parallel for reduction(+ : s) schedule(static)
  for (int64_t i = 0; i < n; ++i) { const double d = (double)y[i] - t[i]; s += d * d; }
  return s / (double)n;
}
/* One bias-corrected Adam step (no weight decay); step counts from 1. */
void orc_adam(float* w, float* m, float* v, const float* g, int64_t n, float lr, float b1,
              float b2, float eps, int64_t step) {
  const double c1 = 1.0 - pow((double)b1, (double)step), c2 = 1.0 - pow((double)b2, (double)step);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    m[i] = b1 * m[i] + (1.0f - b1) * g[i];
    v[i] = b2 * v[i] + (1.0f - b2) * g[i] * g[i];
    const double mh = m[i] / c1, vh = v[i] / c2;
    w[i] = (float)(w[i] - lr * mh / (sqrt(vh) + eps));
  }
}
/* Sum-allreduce restated over `world` host buffers: every buffer ends holding the sum
 * taken in rank order (rank 0 first). */
void orc_all_reduce(float** bufs, int world, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float s = bufs[0][i];
    for (int r = 1; r < world; ++r) s += bufs[r][i];
    for (int r = 0; r < world; ++r) bufs[r][i] = s;
  }
}
int orc_num_threads(void) { return omp_get_max_threads(); }
/* torchrun exports OMP_NUM_THREADS=1 to its workers; the timed CPU baseline asks for the
 * cores the process may actually use instead. */
void orc_set_num_threads(int n) { if (n > 0) omp_set_num_threads(n); }
