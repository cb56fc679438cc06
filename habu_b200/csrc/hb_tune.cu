// Autotune entry point: times every candidate configuration of an operator for one
// problem shape on the device, keeps the winner in the context's cache and persists the
// cache as one text line per entry (format v2):
//   matmul    <dtype> <m> <n> <k> <layout> <epilogue> sm<count> <gpu> = cluster <c> tile <m>x<n>x<k> stages <s> raster <r> ms <t>
//   skinny    ...same key fields...                                   = grid <ctas> kps <k-blocks per stage> ms <t>
//   attention <dtype> <batch*heads> <seq> <head_dim> <causal> <q per kv head> sm<count> <gpu> = persistent <0|1> ms <t>
// (m, n, k are the shapes one GPU computes, so a tensor-parallel shard has its own line).
// A choice is written by its properties, not by its index in the library's table, so a cache
// survives a library whose table has grown; the key carries the GPU's name as well as its SM
// count, so a file copied to another part is not applied there.  Version-1 files (index-valued
// lines, no GPU name) are still read: their indices are translated through the version-1 table.
#include <stdio.h>
#include <string.h>

#include "hb_internal.h"

int hb_gemm_num_configs();
void hb_gemm_config_describe(int id, hb_tune_result* out);
bool hb_gemm_config_supports(int id, const hb_gemm_args& a);
int hb_gemm_find_config(int cluster, int tile_n, int tile_k, int stages, int raster_group);
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

const char* op_name(int op) { return op == HB_OP_MATMUL ? "matmul" : op == HB_OP_SKINNY ? "skinny" : "attention"; }

}  // namespace

std::string hb_tune_key(const hb_op_desc& d, int sm_count, const std::string& gpu) {
  char buf[256];
  snprintf(buf, sizeof(buf), "%s %s %lld %lld %lld %d %d sm%d %s", op_name(d.op), d.dtype == HB_BF16 ? "bf16" : "f32",
           (long long)d.m, (long long)d.n, (long long)d.k, d.layout, d.epilogue, sm_count, gpu.c_str());
  return buf;
}

int hb_gemm_pick_config(hb_ctx* ctx, const hb_gemm_args& a) {
  hb_op_desc d;
  memset(&d, 0, sizeof(d));
  d.op = HB_OP_MATMUL; d.dtype = HB_BF16;
  d.m = a.M; d.n = a.N; d.k = a.K;
  d.layout = (a.a_mn_major ? 1 : 0) | (a.b_mn_major ? 2 : 0);
  d.epilogue = a.epilogue;
  auto it = ctx->tune_cache.find(hb_tune_key(d, ctx->sm_count, ctx->gpu_name));
  if (it != ctx->tune_cache.end() && it->second.config_id >= 0 && it->second.config_id < hb_gemm_num_configs())
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
  int best = 0, seen_n = 0;
  for (int id = 0; id < n; ++id) {
    hb_tune_result r;
    hb_gemm_config_describe(id, &r);
    if (r.raster_group != 8 || r.cluster != 1 || r.tile_n == seen_n) continue;   // the first variant of each width
    seen_n = r.tile_n;
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
    hb_gemm_skinny_plan(sm_count, a.M, a.N, a.K, 0, 0, &grid, &max_seg, &floats, &tiles);
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

namespace {

// Times `fn` (one launch per call) after two warm-up launches; HB_OK and the mean of `reps`.
template <typename F>
hb_status time_launches(hb_ctx* ctx, cudaEvent_t e0, cudaEvent_t e1, int reps, F fn, float* ms) {
  hb_status st = HB_OK;
  for (int w = 0; w < 2; ++w)
    if ((st = fn()) != HB_OK) return st;
  cudaEventRecord(e0, ctx->stream);
  for (int r = 0; r < reps; ++r) fn();
  cudaEventRecord(e1, ctx->stream);
  if ((st = hb_sync(ctx)) != HB_OK) return st;
  cudaEventElapsedTime(ms, e0, e1);
  *ms /= reps;
  return HB_OK;
}

// Attention: the two instantiations (one work unit per CTA; persistent work queue) on
// synthetic Q, K, V of the described shape.
hb_status autotune_attention(hb_ctx* ctx, const hb_op_desc* desc, const std::string& key, hb_tune_result* out) {
  const int64_t B = desc->m, S = desc->n, D = desc->k;
  const int64_t Hq = (desc->epilogue >> 16) & 0xffff, Hkv = desc->epilogue & 0xffff;
  if (B <= 0 || S <= 0 || D != 128 || Hq <= 0 || Hkv <= 0 || Hq % Hkv)
    return hb_fail(ctx, HB_ERR_INVALID, "autotune: attention wants m = batch, n = seq, k = 128, epilogue = q_heads << 16 | kv_heads");
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  const size_t q_b = up((size_t)B * S * Hq * D * 2), kv_b = up((size_t)B * S * Hkv * D * 2);
  void* base = nullptr;
  hb_status st = hb_get_scratch(ctx, HB_SCRATCH_TUNE, 2 * q_b + 2 * kv_b, &base);
  if (st != HB_OK) return st;
  char* dQ = static_cast<char*>(base);
  char *dK = dQ + q_b, *dV = dK + kv_b, *dO = dV + kv_b;
  fill_bf16_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(reinterpret_cast<uint16_t*>(dQ), (q_b + 2 * kv_b) / 2, 0x48414255u);
  ctx->launches++;
  auto mk = [&](char* ptr, int64_t heads) {
    hb_tensor t = {ptr, HB_BF16, 4, {B, S, heads, D}, {S * heads * D, heads * D, D, 1}};
    return t;
  };
  hb_tensor tQ = mk(dQ, Hq), tK = mk(dK, Hkv), tV = mk(dV, Hkv), tO = mk(dO, Hq);
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess)
    return hb_fail(ctx, HB_ERR_CUDA, "autotune: cannot create events");
  int best = -1;
  float best_ms = 0.f;
  for (int persist = 0; persist < 2 && st == HB_OK; ++persist) {
    hb_attn_opts o = {desc->layout ? 1 : 0, 0.08838834764831845f, nullptr, persist};
    float ms = 0.f;
    st = time_launches(ctx, e0, e1, 5, [&] { return hb_attention(ctx, &tQ, &tK, &tV, &tO, &o); }, &ms);
    if (st == HB_OK && (best < 0 || ms < best_ms)) { best = persist; best_ms = ms; }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (st != HB_OK) return st;
  ctx->tune_cache[key] = hb_tune_entry{best, best_ms, 0, 0};
  out->config_id = best;
  out->tile_m = 256; out->tile_n = 128; out->tile_k = 128; out->stages = 2; out->cluster = 1;
  out->ms = best_ms;
  const double flop = 4.0 * B * Hq * S * S * D * (desc->layout ? 0.5 : 1.0);
  out->tflops = (float)(flop / (best_ms * 1e-3) / 1e12);
  return HB_OK;
}

}  // namespace

// The attention node's cached choice: 0 = one unit per CTA, 1 = persistent, -1 = none cached.
int hb_attention_cached_choice(hb_ctx* ctx, int64_t batch, int64_t seq, int64_t hq, int64_t hkv, int causal) {
  hb_op_desc d;
  memset(&d, 0, sizeof(d));
  d.op = HB_OP_ATTENTION; d.dtype = HB_BF16;
  d.m = batch; d.n = seq; d.k = 128; d.layout = causal ? 1 : 0; d.epilogue = (int32_t)((hq << 16) | hkv);
  auto it = ctx->tune_cache.find(hb_tune_key(d, ctx->sm_count, ctx->gpu_name));
  return it == ctx->tune_cache.end() ? -1 : it->second.config_id;
}

// The stream-K kernel's cached (grid, k-blocks per stage), or false.
bool hb_skinny_cached_choice(hb_ctx* ctx, const hb_gemm_args& a, int* grid, int* kps) {
  hb_op_desc d;
  memset(&d, 0, sizeof(d));
  d.op = HB_OP_SKINNY; d.dtype = HB_BF16;
  d.m = a.M; d.n = a.N; d.k = a.K;
  auto it = ctx->tune_cache.find(hb_tune_key(d, ctx->sm_count, ctx->gpu_name));
  if (it == ctx->tune_cache.end()) return false;
  *grid = it->second.p0;
  *kps = it->second.p1;
  return *grid >= 1 && (*kps == 1 || *kps == 2 || *kps == 4);
}

extern "C" hb_status hb_autotune(hb_ctx* ctx, const hb_op_desc* desc, int32_t mode,
                                 hb_tune_result* out) {
  if (!ctx || !desc || !out) return HB_ERR_INVALID;
  if (desc->op != HB_OP_MATMUL && desc->op != HB_OP_ATTENTION)
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "autotune: unknown operator %d", desc->op);
  if (desc->dtype != HB_BF16)
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "autotune: only the bf16 kernels have more than one configuration");
  hb_op_desc d = *desc;
  hb_gemm_args g;
  memset(&g, 0, sizeof(g));
  bool skinny = false;
  if (d.op == HB_OP_MATMUL) {
    if (d.m <= 0 || d.n <= 0 || d.k <= 0 || (d.k & 7)) return hb_fail(ctx, HB_ERR_INVALID, "autotune: bad matmul shape");
    g.M = d.m; g.N = d.n; g.K = d.k;
    g.a_mn_major = d.layout & 1; g.b_mn_major = (d.layout >> 1) & 1;
    g.epilogue = d.epilogue;
    skinny = hb_gemm_skinny_applicable(g);       // M <= 64: the stream-K kernel, tuned over grid and k-blocks per stage
    if (skinny) d.op = HB_OP_SKINNY;
  }
  const std::string key = hb_tune_key(d, ctx->sm_count, ctx->gpu_name);
  memset(out, 0, sizeof(*out));
  if (mode == HB_TUNE_CACHED) {
    auto it = ctx->tune_cache.find(key);
    if (it == ctx->tune_cache.end())
      return hb_fail(ctx, HB_ERR_NOT_FOUND, "autotune: no cached choice for '%s'", key.c_str());
    if (d.op == HB_OP_MATMUL) {
      hb_gemm_config_describe(it->second.config_id, out);
      out->tflops = (float)(2.0 * d.m * d.n * d.k / (it->second.ms * 1e-3) / 1e12);
    } else if (d.op == HB_OP_SKINNY) {
      out->config_id = -1; out->tile_m = 128; out->tile_n = 64; out->tile_k = 64 * it->second.p1; out->cluster = 1;
      out->split_k = it->second.p0;
      out->tflops = (float)(2.0 * d.m * d.n * d.k / (it->second.ms * 1e-3) / 1e12);
    } else {
      out->config_id = it->second.config_id;
    }
    out->ms = it->second.ms;
    return HB_OK;
  }
  if (mode != HB_TUNE_SEARCH) return hb_fail(ctx, HB_ERR_INVALID, "autotune: unknown mode %d", mode);
  if (d.op == HB_OP_ATTENTION) return autotune_attention(ctx, &d, key, out);

  const int64_t M = d.m, N = d.n, K = d.k;
  const int64_t NC = d.epilogue == HB_EPI_SWIGLU ? N / 2 : N;
  const int a_mn = g.a_mn_major, b_mn = g.b_mn_major;
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

  g.A = dA; g.B = dB; g.C = dC;
  g.lda = a_mn ? M : K;
  g.ldb = b_mn ? N : K;
  g.ldc = NC;
  if (d.epilogue == HB_EPI_RESIDUAL) { g.residual = dR; g.ldr = N; }
  if ((g.lda & 7) || (g.ldb & 7))
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "autotune: leading dimensions must be multiples of 8");

  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess)
    return hb_fail(ctx, HB_ERR_CUDA, "autotune: cannot create events");
  const int reps = 5;
  float best_ms = 0.f;
  if (skinny) {
    // grid: every SM, or fewer CTAs with longer K ranges; k-blocks per ring stage: 1, 2 or 4
    int best_grid = 0, best_kps = 0;
    const int sm = ctx->sm_count;
    const int grids[] = {sm, sm - sm / 8, sm - sm / 4, sm / 2};
    for (int gi = 0; gi < 4 && st == HB_OK; ++gi)
      for (int kps = 1; kps <= 4 && st == HB_OK; kps *= 2) {
        float ms = 0.f;
        st = time_launches(ctx, e0, e1, reps, [&] { return hb_launch_gemm_skinny_cfg(ctx, g, grids[gi], kps); }, &ms);
        if (st == HB_OK && (best_grid == 0 || ms < best_ms)) { best_grid = grids[gi]; best_kps = kps; best_ms = ms; }
      }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (st != HB_OK) return st;
    ctx->tune_cache[key] = hb_tune_entry{-1, best_ms, best_grid, best_kps};
    out->config_id = -1; out->tile_m = 128; out->tile_n = 64; out->tile_k = 64 * best_kps; out->cluster = 1;
    out->split_k = best_grid;
  } else {
    int best = -1;
    for (int id = 0; id < hb_gemm_num_configs() && st == HB_OK; ++id) {
      if (!hb_gemm_config_supports(id, g)) continue;
      float ms = 0.f;
      st = time_launches(ctx, e0, e1, reps, [&] { return hb_launch_gemm_bf16(ctx, g, id); }, &ms);
      if (st == HB_OK && (best < 0 || ms < best_ms)) { best = id; best_ms = ms; }
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (st != HB_OK) return st;
    ctx->tune_cache[key] = hb_tune_entry{best, best_ms, 0, 0};
    hb_gemm_config_describe(best, out);
  }
  out->ms = best_ms;
  out->tflops = (float)(2.0 * M * N * K / (best_ms * 1e-3) / 1e12);
  return HB_OK;
}

extern "C" hb_status hb_tune_cache_save(hb_ctx* ctx, const char* path) {
  if (!ctx || !path) return HB_ERR_INVALID;
  FILE* f = fopen(path, "w");
  if (!f) return hb_fail(ctx, HB_ERR_NOT_FOUND, "tune cache: cannot open '%s' for writing", path);
  fprintf(f, "# habu_b200 autotune cache v2\n");
  for (const auto& kv : ctx->tune_cache) {
    const hb_tune_entry& e = kv.second;
    if (kv.first.compare(0, 7, "matmul ") == 0) {
      if (e.config_id < 0 || e.config_id >= hb_gemm_num_configs()) continue;
      hb_tune_result r;
      hb_gemm_config_describe(e.config_id, &r);
      fprintf(f, "%s = cluster %d tile %dx%dx%d stages %d raster %d ms %.6f\n", kv.first.c_str(), r.cluster, r.tile_m,
              r.tile_n, r.tile_k, r.stages, r.raster_group, e.ms);
    } else if (kv.first.compare(0, 7, "skinny ") == 0) {
      fprintf(f, "%s = grid %d kps %d ms %.6f\n", kv.first.c_str(), e.p0, e.p1, e.ms);
    } else {
      fprintf(f, "%s = persistent %d ms %.6f\n", kv.first.c_str(), e.config_id, e.ms);
    }
  }
  fclose(f);
  return HB_OK;
}

extern "C" hb_status hb_tune_cache_load(hb_ctx* ctx, const char* path) {
  if (!ctx || !path) return HB_ERR_INVALID;
  FILE* f = fopen(path, "r");
  if (!f) return hb_fail(ctx, HB_ERR_NOT_FOUND, "tune cache: cannot open '%s'", path);
  // version-1 table: index -> (tile N, stages, raster group, cluster), tile K 64
  static const int v1[16][4] = {{256, 4, 8, 1},  {256, 4, 16, 1}, {256, 4, 4, 1}, {256, 4, 2, 1}, {128, 6, 8, 1}, {128, 6, 16, 1},
                                {128, 6, 4, 1},  {64, 8, 8, 1},   {64, 8, 16, 1}, {256, 6, 8, 2}, {256, 6, 4, 2}, {256, 6, 2, 2},
                                {256, 6, 16, 2}, {256, 7, 8, 2},  {256, 7, 16, 2}, {256, 7, 4, 2}};
  char line[512];
  int lineno = 0, version = 1;
  auto bad = [&]() {
    fclose(f);
    return hb_fail(ctx, HB_ERR_INVALID, "tune cache: syntax error at %s:%d", path, lineno);
  };
  while (fgets(line, sizeof(line), f)) {
    ++lineno;
    if (line[0] == '#') {
      if (strstr(line, "cache v2")) version = 2;
      continue;
    }
    if (line[0] == '\n') continue;
    char* eq = strstr(line, " = ");
    if (!eq) return bad();
    *eq = 0;
    const char* val = eq + 3;
    hb_tune_entry e = {-1, 0.f, 0, 0};
    if (version == 1) {
      int id = -1;
      if (sscanf(val, "%d %f", &id, &e.ms) != 2 || id < 0 || id >= 16) return bad();
      e.config_id = hb_gemm_find_config(v1[id][3], v1[id][0], 64, v1[id][1], v1[id][2]);
      if (e.config_id < 0) continue;
      ctx->tune_cache[std::string(line) + " " + ctx->gpu_name] = e;   // version 1 did not record the GPU
      continue;
    }
    if (strncmp(line, "matmul ", 7) == 0) {
      int cl, tm, tn, tk, stg, ras;
      if (sscanf(val, "cluster %d tile %dx%dx%d stages %d raster %d ms %f", &cl, &tm, &tn, &tk, &stg, &ras, &e.ms) != 7) return bad();
      e.config_id = hb_gemm_find_config(cl, tn, tk, stg, ras);
      if (e.config_id < 0) continue;               // a configuration this build does not have: fall back to the heuristic
    } else if (strncmp(line, "skinny ", 7) == 0) {
      if (sscanf(val, "grid %d kps %d ms %f", &e.p0, &e.p1, &e.ms) != 3) return bad();
    } else if (strncmp(line, "attention ", 10) == 0) {
      if (sscanf(val, "persistent %d ms %f", &e.config_id, &e.ms) != 2) return bad();
    } else {
      return bad();
    }
    ctx->tune_cache[line] = e;
  }
  fclose(f);
  return HB_OK;
}
