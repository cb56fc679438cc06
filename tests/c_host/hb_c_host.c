/*
 * Plain-C host of libhabu_b200.so: the call sequence a foreign-runtime stub makes, with no
 * Python and no C++ in between.  Built with `gcc -std=c99 -pedantic` against the public
 * header only.  Runs the fp32 256^3 matmul of the smallest configuration through the
 * host-buffer entry point and a small causal attention through the device entry points,
 * and checks both against loops written here.  Exit code 0 = all checks passed.
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "habu_b200.h"

#define CHECK(call)                                                                   \
  do {                                                                                \
    hb_status st_ = (call);                                                           \
    if (st_ != HB_OK) {                                                               \
      fprintf(stderr, "%s -> status %d: %s\n", #call, (int)st_, hb_last_error_string(ctx)); \
      return 2;                                                                       \
    }                                                                                 \
  } while (0)

static uint32_t lcg(uint32_t* s) { *s = *s * 1664525u + 1013904223u; return *s; }
static float unit(uint32_t* s) { return (float)(lcg(s) >> 8) * (1.0f / 8388608.0f) - 1.0f; }

/* round-to-nearest-even bf16 */
static uint16_t to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static float from_bf16(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

int main(void) {
  hb_ctx* ctx = NULL;
  uint32_t seed = 0x48414255u;
  int i, j, k;

  if (hb_ctx_create(0, &ctx) != HB_OK) {
    fprintf(stderr, "no sm_100 device: the library has no CPU path\n");
    return 3;
  }

  /* ---- fp32 256 x 256 x 256, B given column-major (as [N, K] row-major) */
  {
    enum { N = 256 };
    float* A = (float*)malloc(sizeof(float) * N * N);
    float* Bt = (float*)malloc(sizeof(float) * N * N);
    float* C = (float*)malloc(sizeof(float) * N * N);
    double worst = 0.0, scale = 0.0;
    for (i = 0; i < N * N; ++i) { A[i] = unit(&seed); Bt[i] = unit(&seed); }
    CHECK(hb_matmul_host(ctx, A, Bt, C, N, N, N, HB_F32));
    for (i = 0; i < N; ++i)
      for (j = 0; j < N; ++j) {
        double acc = 0.0, d;
        for (k = 0; k < N; ++k) acc += (double)A[i * N + k] * (double)Bt[j * N + k];
        d = fabs(acc - (double)C[i * N + j]);
        if (d > worst) worst = d;
        if (fabs(acc) > scale) scale = fabs(acc);
      }
    printf("matmul f32 256^3: max abs err %.3g (max |c| %.3g)\n", worst, scale);
    if (!(worst <= 1e-4 * scale)) return 1;
    free(A); free(Bt); free(C);
  }

  /* ---- causal attention, batch 1, seq 200 (ragged), 2 query heads over 1 KV head, head_dim 128 */
  {
    enum { S = 200, HQ = 2, HKV = 1, D = 128 };
    const float sc = 1.0f / sqrtf((float)D);
    size_t nq = (size_t)S * HQ * D, nkv = (size_t)S * HKV * D;
    uint16_t* q = (uint16_t*)malloc(2 * nq);
    uint16_t* kk = (uint16_t*)malloc(2 * nkv);
    uint16_t* v = (uint16_t*)malloc(2 * nkv);
    uint16_t* o = (uint16_t*)malloc(2 * nq);
    void *dq = NULL, *dk = NULL, *dv = NULL, *dout = NULL;
    hb_tensor tq, tk, tv, to;
    hb_attn_opts opts;
    double worst = 0.0;
    int h, r, c, d;
    for (i = 0; i < (int)nq; ++i) q[i] = to_bf16(unit(&seed) * 2.0f);
    for (i = 0; i < (int)nkv; ++i) { kk[i] = to_bf16(unit(&seed) * 2.0f); v[i] = to_bf16(unit(&seed)); }
    CHECK(hb_alloc(ctx, 2 * nq, &dq));
    CHECK(hb_alloc(ctx, 2 * nkv, &dk));
    CHECK(hb_alloc(ctx, 2 * nkv, &dv));
    CHECK(hb_alloc(ctx, 2 * nq, &dout));
    CHECK(hb_upload(ctx, dq, q, 2 * nq));
    CHECK(hb_upload(ctx, dk, kk, 2 * nkv));
    CHECK(hb_upload(ctx, dv, v, 2 * nkv));
    memset(&tq, 0, sizeof(tq));
    tq.dtype = HB_BF16; tq.rank = 4;
    tq.shape[0] = 1; tq.shape[1] = S; tq.shape[2] = HQ; tq.shape[3] = D;
    tq.stride[0] = (int64_t)S * HQ * D; tq.stride[1] = HQ * D; tq.stride[2] = D; tq.stride[3] = 1;
    to = tq; tk = tq;
    tk.shape[2] = HKV;
    tk.stride[0] = (int64_t)S * HKV * D; tk.stride[1] = HKV * D;
    tv = tk;
    tq.ptr = dq; tk.ptr = dk; tv.ptr = dv; to.ptr = dout;
    memset(&opts, 0, sizeof(opts));
    opts.causal = 1; opts.scale = sc; opts.lse = NULL; opts.config_id = -1;
    CHECK(hb_attention(ctx, &tq, &tk, &tv, &to, &opts));
    CHECK(hb_download(ctx, o, dout, 2 * nq));
    CHECK(hb_sync(ctx));
    for (h = 0; h < HQ; ++h)
      for (r = 0; r < S; ++r) {
        static double p[S];
        double m = -1e300, l = 0.0;
        for (c = 0; c <= r; ++c) {
          double s = 0.0;
          for (d = 0; d < D; ++d) s += (double)from_bf16(q[((size_t)r * HQ + h) * D + d]) * (double)from_bf16(kk[(size_t)c * D + d]);
          p[c] = s * sc;
          if (p[c] > m) m = p[c];
        }
        for (c = 0; c <= r; ++c) { p[c] = exp(p[c] - m); l += p[c]; }
        for (d = 0; d < D; ++d) {
          double acc = 0.0, e;
          for (c = 0; c <= r; ++c) acc += p[c] * (double)from_bf16(v[(size_t)c * D + d]);
          e = fabs(acc / l - (double)from_bf16(o[((size_t)r * HQ + h) * D + d]));
          if (e > worst) worst = e;
        }
      }
    printf("attention bf16 S=200 GQA 2:1: max abs err %.3g\n", worst);
    if (!(worst < 2e-2)) return 1;
    CHECK(hb_free(ctx, dq)); CHECK(hb_free(ctx, dk)); CHECK(hb_free(ctx, dv)); CHECK(hb_free(ctx, dout));
    free(q); free(kk); free(v); free(o);
  }

  /* ---- errors are values: a mismatched inner dimension is reported, nothing is launched */
  {
    hb_tensor a, b, c;
    void* buf = NULL;
    hb_status st;
    CHECK(hb_alloc(ctx, 64 * 64 * 2, &buf));
    memset(&a, 0, sizeof(a));
    a.ptr = buf; a.dtype = HB_BF16; a.rank = 2;
    a.shape[0] = 64; a.shape[1] = 64; a.stride[0] = 64; a.stride[1] = 1;
    b = a; c = a;
    b.shape[0] = 32; b.shape[1] = 64;        /* K = 32 against A's K = 64 */
    st = hb_matmul(ctx, &a, &b, &c, NULL);
    printf("mismatched matmul -> status %d (%s)\n", (int)st, hb_last_error_string(ctx));
    if (st != HB_ERR_INVALID) return 1;
    CHECK(hb_free(ctx, buf));
  }

  if (hb_ctx_destroy(ctx) != HB_OK) return 2;
  printf("OK\n");
  return 0;
}
