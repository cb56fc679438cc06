// Autotune entry point: times every candidate configuration of an operator for one
// problem shape on the device, keeps the winner in the context's cache and persists the
// cache as one text line per entry:
//   <op> <dtype> <m> <n> <k> <layout> <epilogue> sm<count> = <config_id> <ms>
// (m, n, k are the shapes one GPU computes, so a tensor-parallel shard has its own line).
#include <stdio.h>
#include <string.h>

#include "hb_internal.h"

int hb_gemm_num_configs();
void hb_gemm_config_describe(int id, hb_tune_result* out);
bool hb_gemm_config_supports(int id, const hb_gemm_args& a);
int hb_gemm_heuristic_config(int sm_count, int64_t M, int64_t N);

namespace {

__global__ void fill_bf16_kernel(uint16_t* p, size_t n, uint32_t seed) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    uint32_t x = (uint32_t)i * 2654435761u + seed;
    x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
    // bf16 bit patterns in (-0.25, 0.25): sign | exponent 0x7a..0x7c | 7 mantissa bits
    p[i] = (uint16_t)(((x & 1u) << 15) | ((0x7au + ((x >> 1) % 3u)) << 7) | ((x >> 8) & 0x7fu));
  }
}

}  // namespace

std::string hb_tune_key(const hb_op_desc& d, int sm_count, int world) {
  char buf[160];
  (void)world;
  snprintf(buf, sizeof(buf), "%s %s %lld %lld %lld %d %d sm%d",
           d.op == HB_OP_MATMUL ? "matmul" : "attention", d.dtype == HB_BF16 ? "bf16" : "f32",
           (long long)d.m, (long long)d.n, (long long)d.k, d.layout, d.epilogue, sm_count);
  return buf;
}

int hb_gemm_pick_config(hb_ctx* ctx, const hb_gemm_args& a) {
  hb_op_desc d;
  memset(&d, 0, sizeof(d));
  d.op = HB_OP_MATMUL; d.dtype = HB_BF16;
  d.m = a.M; d.n = a.N; d.k = a.K;
  d.layout = (a.a_mn_major ? 1 : 0) | (a.b_mn_major ? 2 : 0);
  d.epilogue = a.epilogue;
  auto it = ctx->tune_cache.find(hb_tune_key(d, ctx->sm_count, ctx->world));
  if (it != ctx->tune_cache.end() && it->second.config_id < hb_gemm_num_configs())
    return it->second.config_id;
  return hb_gemm_heuristic_config(ctx->sm_count, a.M, a.N);
}

// The CTA-pair 256 x 256 tile when there is a tile for every pair of SMs; else the widest
// one-CTA tile that still gives every SM a tile.
int hb_gemm_heuristic_config(int sm_count, int64_t M, int64_t N) {
  const int n = hb_gemm_num_configs();
  if (((M + 255) / 256) * ((N + 255) / 256) >= sm_count / 2) {
    for (int id = 0; id < n; ++id) {
      hb_tune_result r;
      hb_gemm_config_describe(id, &r);
      if (r.cluster == 2 && r.raster_group == 8) return id;
    }
  }
  const int64_t tiles_m = (M + 127) / 128;
  int best = 0;
  for (int id = 0; id < n; ++id) {
    hb_tune_result r;
    hb_gemm_config_describe(id, &r);
    if (r.raster_group != 8 || r.cluster != 1) continue;
    const int64_t tiles = tiles_m * ((N + r.tile_n - 1) / r.tile_n);
    best = id;
    if (tiles >= sm_count) break;
  }
  return best;
}

extern "C" hb_status hb_matmul_default_route(int32_t sm_count, const hb_op_desc* desc, hb_matmul_route* out) {
  if (!desc || !out || sm_count < 1) return HB_ERR_INVALID;
  if (desc->op != HB_OP_MATMUL || desc->dtype != HB_BF16) return HB_ERR_UNSUPPORTED;
  if (desc->m <= 0 || desc->n <= 0 || desc->k <= 0) return HB_ERR_INVALID;
  memset(out, 0, sizeof(*out));
  hb_gemm_args a;
  memset(&a, 0, sizeof(a));
  a.M = desc->m; a.N = desc->n; a.K = desc->k;
  a.a_mn_major = desc->layout & 1; a.b_mn_major = (desc->layout >> 1) & 1;
  a.epilogue = desc->epilogue;
  if (hb_gemm_skinny_applicable(a)) {
    int grid = 0, max_seg = 0, tiles = 0;
    size_t floats = 0;
    hb_gemm_skinny_plan(sm_count, a.M, a.N, a.K, &grid, &max_seg, &floats, &tiles);
    out->kernel = 2;
    out->config_id = -1;
    out->grid = grid; out->tiles = tiles; out->max_segments = max_seg;
    out->scratch_bytes = (int64_t)(floats * sizeof(float));
    return HB_OK;
  }
  hb_tune_result r;
  out->config_id = hb_gemm_heuristic_config(sm_count, a.M, a.N);
  hb_gemm_config_describe(out->config_id, &r);
  out->kernel = r.cluster == 2 ? 1 : 0;
  return HB_OK;
}

extern "C" int32_t hb_matmul_config_count(void) { return hb_gemm_num_configs(); }

extern "C" hb_status hb_matmul_config_info(int32_t config_id, hb_tune_result* out) {
  if (!out || config_id < 0 || config_id >= hb_gemm_num_configs()) return HB_ERR_INVALID;
  memset(out, 0, sizeof(*out));
  hb_gemm_config_describe(config_id, out);
  return HB_OK;
}

extern "C" hb_status hb_autotune(hb_ctx* ctx, const hb_op_desc* desc, int32_t mode,
                                 hb_tune_result* out) {
  if (!ctx || !desc || !out) return HB_ERR_INVALID;
  if (desc->op != HB_OP_MATMUL)
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "autotune: only matmul has more than one configuration");
  if (desc->dtype != HB_BF16)
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "autotune: the fp32 matmul has a single configuration");
  if (desc->m <= 0 || desc->n <= 0 || desc->k <= 0 || (desc->k & 7))
    return hb_fail(ctx, HB_ERR_INVALID, "autotune: bad matmul shape");
  const std::string key = hb_tune_key(*desc, ctx->sm_count, ctx->world);
  memset(out, 0, sizeof(*out));
  if (mode == HB_TUNE_CACHED) {
    auto it = ctx->tune_cache.find(key);
    if (it == ctx->tune_cache.end())
      return hb_fail(ctx, HB_ERR_NOT_FOUND, "autotune: no cached choice for '%s'", key.c_str());
    hb_gemm_config_describe(it->second.config_id, out);
    out->ms = it->second.ms;
    out->tflops = (float)(2.0 * desc->m * desc->n * desc->k / (it->second.ms * 1e-3) / 1e12);
    return HB_OK;
  }
  if (mode != HB_TUNE_SEARCH) return hb_fail(ctx, HB_ERR_INVALID, "autotune: unknown mode %d", mode);

  const int64_t M = desc->m, N = desc->n, K = desc->k;
  const int64_t NC = desc->epilogue == HB_EPI_SWIGLU ? N / 2 : N;
  const int a_mn = desc->layout & 1, b_mn = (desc->layout >> 1) & 1;
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  const size_t a_b = up((size_t)M * K * 2), b_b = up((size_t)N * K * 2), c_b = up((size_t)M * NC * 2);
  void* base = nullptr;
  hb_status st = hb_get_scratch(ctx, HB_SCRATCH_TUNE, a_b + b_b + 2 * c_b, &base);
  if (st != HB_OK) return st;
  char* dA = static_cast<char*>(base);
  char* dB = dA + a_b;
  char* dC = dB + b_b;
  char* dR = dC + c_b;
  fill_bf16_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(
      reinterpret_cast<uint16_t*>(dA), (a_b + b_b + 2 * c_b) / 2, 0x48414255u);
  ctx->launches++;

  hb_gemm_args g;
  memset(&g, 0, sizeof(g));
  g.A = dA; g.B = dB; g.C = dC;
  g.M = M; g.N = N; g.K = K;
  g.a_mn_major = a_mn; g.b_mn_major = b_mn;
  g.lda = a_mn ? M : K;
  g.ldb = b_mn ? N : K;
  g.ldc = NC;
  g.epilogue = desc->epilogue;
  if (desc->epilogue == HB_EPI_RESIDUAL) { g.residual = dR; g.ldr = N; }
  if ((g.lda & 7) || (g.ldb & 7))
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "autotune: leading dimensions must be multiples of 8");

  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess)
    return hb_fail(ctx, HB_ERR_CUDA, "autotune: cannot create events");
  int best = -1;
  float best_ms = 0.f;
  const int reps = 5;
  for (int id = 0; id < hb_gemm_num_configs(); ++id) {
    if (!hb_gemm_config_supports(id, g)) continue;
    for (int w = 0; w < 2; ++w)
      if ((st = hb_launch_gemm_bf16(ctx, g, id)) != HB_OK) break;
    if (st != HB_OK) break;
    cudaEventRecord(e0, ctx->stream);
    for (int r = 0; r < reps; ++r) hb_launch_gemm_bf16(ctx, g, id);
    cudaEventRecord(e1, ctx->stream);
    if ((st = hb_sync(ctx)) != HB_OK) break;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    ms /= reps;
    if (best < 0 || ms < best_ms) { best = id; best_ms = ms; }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (st != HB_OK) return st;
  ctx->tune_cache[key] = hb_tune_entry{best, best_ms};
  hb_gemm_config_describe(best, out);
  out->ms = best_ms;
  out->tflops = (float)(2.0 * M * N * K / (best_ms * 1e-3) / 1e12);
  return HB_OK;
}

extern "C" hb_status hb_tune_cache_save(hb_ctx* ctx, const char* path) {
  if (!ctx || !path) return HB_ERR_INVALID;
  FILE* f = fopen(path, "w");
  if (!f) return hb_fail(ctx, HB_ERR_NOT_FOUND, "tune cache: cannot open '%s' for writing", path);
  fprintf(f, "# habu_b200 autotune cache v1\n");
  for (const auto& kv : ctx->tune_cache)
    fprintf(f, "%s = %d %.6f\n", kv.first.c_str(), kv.second.config_id, kv.second.ms);
  fclose(f);
  return HB_OK;
}

extern "C" hb_status hb_tune_cache_load(hb_ctx* ctx, const char* path) {
  if (!ctx || !path) return HB_ERR_INVALID;
  FILE* f = fopen(path, "r");
  if (!f) return hb_fail(ctx, HB_ERR_NOT_FOUND, "tune cache: cannot open '%s'", path);
  char line[512];
  int lineno = 0;
  while (fgets(line, sizeof(line), f)) {
    ++lineno;
    if (line[0] == '#' || line[0] == '\n') continue;
    char* eq = strstr(line, " = ");
    int id = -1;
    float ms = 0.f;
    if (!eq || sscanf(eq + 3, "%d %f", &id, &ms) != 2 || id < 0) {
      fclose(f);
      return hb_fail(ctx, HB_ERR_INVALID, "tune cache: syntax error at %s:%d", path, lineno);
    }
    *eq = 0;
    ctx->tune_cache[line] = hb_tune_entry{id, ms};
  }
  fclose(f);
  return HB_OK;
}
