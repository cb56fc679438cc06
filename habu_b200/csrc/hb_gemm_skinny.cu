// Skinny (decode-shaped) bf16 GEMM for sm_100a: C[M,N] = A[M,K] . B[K,N] with M <= 64.
// The product is HBM-bound on reading B (N*K*2 bytes), so the kernel is built to keep
// every SM streaming B:
//   * operands are swapped: a 128-row slab of B (stored [N,K], K contiguous) is the MMA's
//     M-side operand and A (padded to a multiple of 16 rows by TMA zero fill) is its N-side
//     operand, so tcgen05.mma runs at M=128, N=16..64 and no tensor-core work is wasted on
//     padding M up to 128;
//   * stream-K: the (tile, k-block) units are cut into one contiguous, equal range per CTA
//     and one persistent CTA runs per SM with an 8..11-stage TMA ring (~200 KB in flight),
//     so every SM streams the same number of bytes and pays one prologue;
//   * a range that covers only part of a tile writes its fp32 partial to scratch; the last
//     range to finish a tile (atomic ticket) adds the partials in k order -- a fixed order,
//     so the result is bit-identical run to run -- rounds to bf16 once and writes C;
//   * programmatic dependent launch: B holds weights, which no kernel of a step writes, so the
//     loader fills the whole ring with B before it waits for the kernel in front of it on the
//     stream (whose output is A, a few KB); in a generation step the weights of the next
//     product stream in while the small kernels between the products (norm, RoPE, attention
//     over the cache, SwiGLU) are still running.  Everything that depends on that kernel -- the
//     A loads, the partials, tickets and C -- comes after the wait.  Only launches whose caller
//     says that B is a weight matrix (HB_MATMUL_WEIGHTS_B) are made that way; any other keeps
//     plain stream order (the wait then returns at once).
// Scratch: tiles * max_segments * 128 * Mpad floats of partials plus one ticket per tile
// (tickets are left at zero by the CTA that consumes them).
// Algorithmic traffic per launch: (N*K + M*K + M*N) * 2 bytes.
#include <stdlib.h>
#include <string.h>

#include "hb_internal.h"
#include "hb_ptx.cuh"

namespace {

using namespace hb;

constexpr int BN_ROWS = 128;   // rows of B per tile (MMA M)
constexpr int BK = 64;
constexpr int MAX_STAGES = 12;
constexpr int SK_THREADS = 192;
constexpr int MAX_MPAD = 64;
constexpr int B_BYTES = BN_ROWS * BK * 2;   // 16 KB

struct SkinnyParams {
  __nv_bfloat16* C;
  float* partial;      // [tile][segment][128][mpad]
  int* tickets;        // [tile]
  int M, N, K;
  int64_t ldc;
  int mpad;            // M rounded up to 16
  int stages;          // ring depth (<= MAX_STAGES)
  int a_bytes;         // bytes of one A stage (mpad * 128)
  int kps;             // 64-wide k-blocks fetched per stage (contiguous bytes per row = 128 * kps)
  int num_kb;          // k-groups (of kps k-blocks) per tile
  int tiles;
  int max_seg;         // partial slots per tile
  int64_t units;       // tiles * num_kb
  int32_t* status;
};

// CTA that owns unit u when `units` are cut into `g` contiguous ranges [c*units/g, (c+1)*units/g).
__device__ __forceinline__ int cta_of(int64_t u, int64_t units, int g) {
  return static_cast<int>(((u + 1) * g - 1) / units);
}

__global__ void __launch_bounds__(SK_THREADS, 1)
hb_gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmA,
                      const SkinnyParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  // layout: B stages | A stages (1 KB aligned each) | barriers | tmem ptr | abort | last flag
  const uint32_t a_box = (static_cast<uint32_t>(p.a_bytes) + 1023u) & ~1023u;
  const uint32_t a_stride = a_box * p.kps;
  const uint32_t b_stride = B_BYTES * p.kps;
  const uint32_t sB = smem_base;
  const uint32_t sA = sB + p.stages * b_stride;
  const uint32_t bar_full = sA + p.stages * a_stride;
  const uint32_t bar_empty = bar_full + MAX_STAGES * 8;
  const uint32_t bar_tfull = bar_empty + MAX_STAGES * 8;
  const uint32_t bar_tempty = bar_tfull + 2 * 8;
  uint8_t* tail = smem + (bar_tempty + 2 * 8 - smem_base);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);
  volatile int* is_last = reinterpret_cast<volatile int*>(tail + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = gridDim.x;
  const int64_t u_begin = p.units * blockIdx.x / g;
  const int64_t u_end = p.units * (blockIdx.x + 1) / g;
  constexpr uint32_t TMEM_COLS = 128;        // two accumulators of up to 64 columns

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *is_last = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + a * 8, 1);
      mbar_init(bar_tempty + a * 8, 128);
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  grid_launch_dependents();     // the next kernel on the stream may begin its own prologue

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      // Ring fill: B (weights) of the first `stages` units before the dependency wait, their A
      // after it.  The slots are empty at start, so no wait on `empty` is needed here.
      const int64_t n_units = u_end - u_begin;
      const int fill = static_cast<int>(n_units < p.stages ? n_units : p.stages);
      for (int i = 0; i < fill; ++i) {
        const int64_t u = u_begin + i;
        const int tile = static_cast<int>(u / p.num_kb);
        const int kb = static_cast<int>(u % p.num_kb);
        mbar_arrive_expect_tx(bar_full + i * 8, (B_BYTES + p.a_bytes) * p.kps);
        for (int x = 0; x < p.kps; ++x)
          tma_load_2d(sB + i * b_stride + x * B_BYTES, &tmB, bar_full + i * 8, (kb * p.kps + x) * BK, tile * BN_ROWS);
      }
      grid_dependency_wait();
      for (int i = 0; i < fill; ++i) {
        const int kb = static_cast<int>((u_begin + i) % p.num_kb);
        for (int x = 0; x < p.kps; ++x)
          tma_load_2d(sA + i * a_stride + x * a_box, &tmA, bar_full + i * 8, (kb * p.kps + x) * BK, 0);
      }
      s = fill == p.stages ? 0 : fill;
      phase = fill == p.stages ? 1 : 0;
      for (int64_t u = u_begin + fill; u < u_end; ++u) {
        const int tile = static_cast<int>(u / p.num_kb);
        const int kb = static_cast<int>(u % p.num_kb);
        if (!mbar_wait(bar_empty + s * 8, phase ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(bar_full + s * 8, (B_BYTES + p.a_bytes) * p.kps);
        for (int x = 0; x < p.kps; ++x) {   // consecutive k-blocks: 128 * kps contiguous bytes per row
          tma_load_2d(sB + s * b_stride + x * B_BYTES, &tmB, bar_full + s * 8, (kb * p.kps + x) * BK, tile * BN_ROWS);
          tma_load_2d(sA + s * a_stride + x * a_box, &tmA, bar_full + s * 8, (kb * p.kps + x) * BK, 0);
        }
        if (++s == p.stages) { s = 0; phase ^= 1; }
      }
      if (!ok && p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_SPLITK; p.status[2] = 1; }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_bf16(BN_ROWS, p.mpad, 0, 0);
      int s = 0;
      uint32_t phase = 0;
      int seg = 0;
      bool ok = true;
      for (int64_t u = u_begin; u < u_end && ok; ++seg) {
        const int kb0 = static_cast<int>(u % p.num_kb);
        const int64_t left = u_end - u;
        const int nkb = static_cast<int>(left < p.num_kb - kb0 ? left : p.num_kb - kb0);
        const int acc = seg & 1;
        if (!mbar_wait(bar_tempty + acc * 8, ((seg >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (int i = 0; i < nkb; ++i) {
          if (!mbar_wait(bar_full + s * 8, phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          for (int x = 0; x < p.kps; ++x) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_ss<1>(tmem_base + acc * 64, umma_desc_k_sw128(sB + s * b_stride + x * B_BYTES + k * 32),
                         umma_desc_k_sw128(sA + s * a_stride + x * a_box + k * 32), idesc, (i | x | k) != 0 ? 1u : 0u);
          }
          umma_commit<1>(bar_empty + s * 8);
          if (++s == p.stages) { s = 0; phase ^= 1; }
        }
        if (ok) umma_commit<1>(bar_tfull + acc * 8);
        u += nkb;
      }
      if (!ok && p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_SPLITK; p.status[2] = 2; }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int q = warp & 3;
    const int r = q * 32 + lane;                 // row of the B slab = output column n0 + r
    const int etid = (warp - 2) * 32 + lane;     // 0..127
    bool ok = true;
    int seg = 0;
    grid_dependency_wait();                      // partials, tickets and C may still be in use by the kernel in front
    for (int64_t u = u_begin; u < u_end; ++seg) {
      const int tile = static_cast<int>(u / p.num_kb);
      const int kb0 = static_cast<int>(u % p.num_kb);
      const int64_t left = u_end - u;
      const int nkb = static_cast<int>(left < p.num_kb - kb0 ? left : p.num_kb - kb0);
      u += nkb;
      const int acc_i = seg & 1;
      if (ok) ok = mbar_wait(bar_tfull + acc_i * 8, (seg >> 1) & 1, abort_flag);
      float acc[MAX_MPAD];
#pragma unroll
      for (int i = 0; i < MAX_MPAD; ++i) acc[i] = 0.f;
      if (ok) {
        tc_fence_after();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc_i * 64;
#pragma unroll
        for (int c = 0; c < MAX_MPAD / 16; ++c) {
          if (c * 16 < p.mpad) {
            uint32_t v[16];
            tmem_ld_32x16(t_row + c * 16, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[c * 16 + i] = __uint_as_float(v[i]);
          }
        }
        tc_fence_before();
        mbar_arrive(bar_tempty + acc_i * 8);    // the accumulator is in registers: free it
      }
      const bool whole = nkb == p.num_kb;
      bool write_out = whole;
      if (!whole) {
        // position of this range among the ranges that share the tile, in k order
        const int64_t t0 = static_cast<int64_t>(tile) * p.num_kb;
        const int c_first = cta_of(t0, p.units, g);
        const int c_last = cta_of(t0 + p.num_kb - 1, p.units, g);
        const int nseg = c_last - c_first + 1;
        const int slot = static_cast<int>(blockIdx.x) - c_first;
        float* base = p.partial + (static_cast<int64_t>(tile) * p.max_seg) * BN_ROWS * p.mpad;
        float* mine = base + (static_cast<int64_t>(slot) * BN_ROWS + r) * p.mpad;
#pragma unroll
        for (int c = 0; c < MAX_MPAD / 4; ++c)
          if (c * 4 < p.mpad)
            *reinterpret_cast<float4*>(mine + c * 4) = make_float4(acc[c * 4], acc[c * 4 + 1], acc[c * 4 + 2], acc[c * 4 + 3]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (etid == 0) {
          const int ticket = atomicAdd(p.tickets + tile, 1);
          const int last = ticket == nseg - 1;
          if (last) p.tickets[tile] = 0;         // leave the ticket ready for the next launch
          *is_last = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        write_out = *is_last != 0;
        if (write_out) {
          __threadfence();
#pragma unroll
          for (int i = 0; i < MAX_MPAD; ++i) acc[i] = 0.f;
          for (int sidx = 0; sidx < nseg; ++sidx) {   // k order: bit-identical run to run
            const float* src = base + (static_cast<int64_t>(sidx) * BN_ROWS + r) * p.mpad;
#pragma unroll
            for (int c = 0; c < MAX_MPAD / 4; ++c)
              if (c * 4 < p.mpad) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(src + c * 4));
                acc[c * 4] += v.x; acc[c * 4 + 1] += v.y; acc[c * 4 + 2] += v.z; acc[c * 4 + 3] += v.w;
              }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // is_last is rewritten by the next range
      }
      if (write_out && ok) {
        const int n = tile * BN_ROWS + r;
        if (n < p.N) {
#pragma unroll
          for (int m = 0; m < MAX_MPAD; ++m)
            if (m < p.M) p.C[static_cast<int64_t>(m) * p.ldc + n] = __float2bfloat16_rn(acc[m]);
        }
      }
    }
    if (!ok && p.status && lane == 0) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_SPLITK; p.status[2] = 3; }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}

// k-blocks per ring stage: the given value if valid, else HB_SKINNY_KPS, else 2.
int skinny_kps(int want) {
  if (want == 1 || want == 2 || want == 4) return want;
  int k = 2;
  if (const char* e = getenv("HB_SKINNY_KPS")) { const int v = atoi(e); if (v == 1 || v == 2 || v == 4) k = v; }
  return k;
}
int skinny_stages(int mpad, int kps) {
  const int stage = kps * (B_BYTES + ((mpad * 128 + 1023) & ~1023));
  int st = (200 * 1024) / stage;
  return st > MAX_STAGES ? MAX_STAGES : st;
}
int skinny_smem_bytes(int mpad, int kps) {
  const int stage = kps * (B_BYTES + ((mpad * 128 + 1023) & ~1023));
  return skinny_stages(mpad, kps) * stage + (2 * MAX_STAGES + 4) * 8 + 16 + 1024;
}

}  // namespace

bool hb_gemm_skinny_applicable(const hb_gemm_args& a) {
  return a.M <= MAX_MPAD && !a.a_mn_major && !a.b_mn_major && a.epilogue == HB_EPI_NONE && a.N >= 256;
}

// Chooses the grid and reports the scratch the launch needs: `grid` persistent CTAs, at
// most `max_seg` ranges per tile, `partial_floats` floats of partials, `tiles` tickets.
// `grid_cap` (<= 0: one CTA per SM, or HB_SKINNY_CTAS) and `kps` (<= 0: default) are the two
// axes the autotuner searches.
void hb_gemm_skinny_plan(int sm_count, int64_t M, int64_t N, int64_t K, int grid_cap, int kps_in, int* grid, int* max_seg,
                         size_t* partial_floats, int* tiles) {
  const int t = (int)((N + BN_ROWS - 1) / BN_ROWS);
  const int kps = skinny_kps(kps_in);
  const int num_kb = (int)((K + BK * kps - 1) / (BK * kps));      // k-groups per tile
  const int mpad = (int)((M + 15) / 16) * 16;
  const int64_t units = (int64_t)t * num_kb;
  int g = sm_count;
  if (grid_cap >= 1) g = grid_cap < sm_count ? grid_cap : sm_count;
  else if (const char* e = getenv("HB_SKINNY_CTAS")) { const int v = atoi(e); if (v >= 1) g = v; }
  if (units / 4 < g) g = (int)(units / 4 > 0 ? units / 4 : 1);     // at least 4 k-groups per CTA
  const int64_t per = units / g;                                     // shortest range
  int ms = (int)((num_kb + per - 1) / per) + 1;
  if (ms > g) ms = g;
  *grid = g;
  *max_seg = ms;
  *tiles = t;
  *partial_floats = (size_t)t * ms * BN_ROWS * mpad;
}

hb_status hb_launch_gemm_skinny_raw(hb_ctx* ctx, cudaStream_t stream, const hb_gemm_args& a, float* partial, int* tickets,
                                    int grid, int max_seg, int tiles, int kps, int32_t* status) {
  CUtensorMap tmA, tmB;
  const int mpad = (int)((a.M + 15) / 16) * 16;
  {
    uint64_t dims[2] = {(uint64_t)a.K, (uint64_t)a.N};
    uint64_t strides[1] = {(uint64_t)a.ldb * 2};
    uint32_t box[2] = {BK, BN_ROWS};
    hb_status st = hb_make_tensor_map(ctx, &tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.B, dims, strides, box,
                                      CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != HB_OK) return st;
  }
  {
    uint64_t dims[2] = {(uint64_t)a.K, (uint64_t)a.M};
    uint64_t strides[1] = {(uint64_t)a.lda * 2};
    uint32_t box[2] = {BK, (uint32_t)mpad};
    hb_status st = hb_make_tensor_map(ctx, &tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.A, dims, strides, box,
                                      CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != HB_OK) return st;
  }
  SkinnyParams p;
  memset(&p, 0, sizeof(p));
  p.C = static_cast<__nv_bfloat16*>(a.C);
  p.partial = partial;
  p.tickets = tickets;
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.ldc = a.ldc;
  p.mpad = mpad;
  p.kps = skinny_kps(kps);
  p.stages = skinny_stages(mpad, p.kps);
  p.a_bytes = mpad * 128;
  p.num_kb = (int)((a.K + BK * p.kps - 1) / (BK * p.kps));
  p.tiles = tiles;
  p.max_seg = max_seg;
  p.units = (int64_t)tiles * p.num_kb;
  p.status = status;
  // the attribute is per device: one flag for each device this process launches on
  static bool attr_set_dev[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  bool& attr_set = attr_set_dev[dev & 63];
  if (!attr_set) {
    int most = 0;
    for (int m = 16; m <= MAX_MPAD; m += 16)
      for (int k = 1; k <= 4; k *= 2) most = skinny_smem_bytes(m, k) > most ? skinny_smem_bytes(m, k) : most;
    cudaError_t e = cudaFuncSetAttribute(hb_gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaFuncSetAttribute(skinny gemm)");
    attr_set = true;
  }
  // A launch whose B is a weight matrix may overlap the tail of the kernel in front of it on the
  // stream (programmatic dependent launch: see the header of this file); every other launch, and
  // the context-free static entry point, keeps plain stream order.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(SK_THREADS);
  cfg.dynamicSmemBytes = skinny_smem_bytes(mpad, p.kps);
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  bool pdl = ctx != nullptr && a.b_is_weights;
  if (const char* e = getenv("HB_SKINNY_PDL")) pdl = pdl && atoi(e) != 0;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t le = cudaLaunchKernelEx(&cfg, hb_gemm_skinny_kernel, tmB, tmA, p);
  if (le != cudaSuccess) return hb_check_cuda(ctx, le, "skinny gemm launch");
  return hb_check_cuda(ctx, cudaGetLastError(), "skinny gemm launch");
}

hb_status hb_launch_gemm_skinny_cfg(hb_ctx* ctx, const hb_gemm_args& a, int grid_cap, int kps) {
  int grid, max_seg, tiles;
  size_t floats;
  hb_gemm_skinny_plan(ctx->sm_count, a.M, a.N, a.K, grid_cap, kps, &grid, &max_seg, &floats, &tiles);
  if (tiles > HB_MAX_SPLITK_TILES) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "matmul: N too large for the split-K path");
  void* ws = nullptr;
  hb_status st = hb_get_scratch(ctx, HB_SCRATCH_WORKSPACE, floats * sizeof(float), &ws);
  if (st != HB_OK) return st;
  st = hb_launch_gemm_skinny_raw(ctx, ctx->stream, a, static_cast<float*>(ws), ctx->d_tickets, grid, max_seg, tiles, kps,
                                 ctx->d_status);
  if (st == HB_OK) ctx->launches++;
  return st;
}

// The autotune cache's (grid, k-blocks per stage) for this shape when it has one.
hb_status hb_launch_gemm_skinny(hb_ctx* ctx, const hb_gemm_args& a) {
  int grid_cap = 0, kps = 0;
  if (!hb_skinny_cached_choice(ctx, a, &grid_cap, &kps)) { grid_cap = 0; kps = 0; }
  return hb_launch_gemm_skinny_cfg(ctx, a, grid_cap, kps);
}

// ---------------------------------------------------------------------------------------
// hb_matmul_skinny_static: the skinny GEMM for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a
// product: a real-time serving loop that forbids allocator locks and the implicit device
// synchronisation cudaMalloc/cudaFree can cause; a foreign-runtime finaliser or signal
// path (an OCaml stub running under the runtime lock, say) where a blocking driver call is
// not allowed; a process whose memory budget was fixed at start-up and handed out in full.
// For them the split-K scratch lives in the file-scope arrays below instead of in a
// context-owned buffer.  Every GPU that loads the library carries these arrays (about
// 4 MiB) until the process exits.
//
// Limits: partials ceil(N/128) * segments * 128 * Mpad <= HB_STATIC_MAX_PARTIAL_FLOATS (segments
// = ranges of K that can share one tile, 4 at N=K=8192 on 148 SMs) and ceil(N/128) <=
// HB_STATIC_MAX_TILES; larger problems are refused with HB_ERR_UNSUPPORTED.
// The first call on a device resolves the arrays' device addresses and sets the kernel's
// shared-memory attribute; it should come before any stream capture.
// All calls share the arrays: two calls that overlap on the GPU (different streams) race
// on the partials and tickets, so serialise them.  The tickets must start at zero and are
// cleared on the stream before every launch; the partials need no clearing because every
// slot read is written first in the same launch.
// ---------------------------------------------------------------------------------------
#include <mutex>

namespace {

constexpr size_t HB_STATIC_MAX_PARTIAL_FLOATS = size_t(1) << 20;   // 4 MiB
constexpr int HB_STATIC_MAX_TILES = 1024;

static __device__ __align__(256) float g_static_partial[HB_STATIC_MAX_PARTIAL_FLOATS];
static __device__ __align__(256) int g_static_tickets[HB_STATIC_MAX_TILES];
static __device__ __align__(256) int32_t g_static_status[4];

struct StaticDev {
  bool ready = false;
  float* partial = nullptr;
  int* tickets = nullptr;
  int32_t* status = nullptr;
  int sm_count = 0;
};
StaticDev g_static_dev[64];
std::mutex g_static_mu;
thread_local char g_static_err[256] = "";

hb_status static_fail(hb_status code, const char* msg, const char* detail = "") {
  snprintf(g_static_err, sizeof(g_static_err), "%s%s", msg, detail);
  return code;
}

// In host code the array names above are host-side stand-ins, not device addresses; the
// address a kernel can use comes from cudaGetSymbolAddress, per device, with that device
// current.
// cudaGetSymbolAddress (like the status copies of hb_static_status) acts on the calling
// thread's CURRENT device, so a `device` that is not current is refused here, for every
// entry point: otherwise another GPU's addresses would be cached under `device`.
hb_status static_setup(int device, StaticDev** out) {
  if (device < 0 || device >= 64) return static_fail(HB_ERR_INVALID, "skinny_static: device index out of range");
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess || cur != device) {
    cudaGetLastError();
    return static_fail(HB_ERR_INVALID, "skinny_static: `device` must be the current CUDA device of the calling thread");
  }
  std::lock_guard<std::mutex> lock(g_static_mu);
  StaticDev& d = g_static_dev[device];
  if (!d.ready) {
    cudaError_t e;
    if ((e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.partial), g_static_partial)) != cudaSuccess ||
        (e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.tickets), g_static_tickets)) != cudaSuccess ||
        (e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status), g_static_status)) != cudaSuccess)
      return static_fail(HB_ERR_CUDA, "skinny_static: cudaGetSymbolAddress: ", cudaGetErrorString(e));
    int major = 0;
    if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess)
      return static_fail(HB_ERR_CUDA, "skinny_static: cudaDeviceGetAttribute: ", cudaGetErrorString(e));
    if (major != 10) return static_fail(HB_ERR_UNSUPPORTED, "skinny_static: an sm_100 GPU is required");
    d.ready = true;
  }
  *out = &d;
  return HB_OK;
}

}  // namespace

extern "C" const char* hb_static_last_error(void) { return g_static_err; }

extern "C" hb_status hb_matmul_skinny_static(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                             int32_t device, void* cuda_stream) {
  g_static_err[0] = 0;
  if (!A || !B || !C) return static_fail(HB_ERR_INVALID, "skinny_static: null pointer");
  if (M <= 0 || N <= 0 || K <= 0) return static_fail(HB_ERR_INVALID, "skinny_static: empty dimension");
  if (M > MAX_MPAD) return static_fail(HB_ERR_UNSUPPORTED, "skinny_static: M must be at most 64");
  if (K % 8 || N % 8) return static_fail(HB_ERR_UNSUPPORTED, "skinny_static: N and K must be multiples of 8");
  if (N > INT32_MAX || K > INT32_MAX) return static_fail(HB_ERR_UNSUPPORTED, "skinny_static: dimension exceeds 2^31-1");
  StaticDev* d = nullptr;
  hb_status st = static_setup(device, &d);
  if (st != HB_OK) return st;
  int grid, max_seg, tiles;
  size_t floats;
  hb_gemm_skinny_plan(d->sm_count, M, N, K, 0, 0, &grid, &max_seg, &floats, &tiles);
  if (tiles > HB_STATIC_MAX_TILES || floats > HB_STATIC_MAX_PARTIAL_FLOATS) {
    char detail[128];
    snprintf(detail, sizeof(detail), "needs %zu partial floats over %d tiles; the static scratch holds %zu floats and %d tiles",
             floats, tiles, HB_STATIC_MAX_PARTIAL_FLOATS, HB_STATIC_MAX_TILES);
    return static_fail(HB_ERR_UNSUPPORTED, "skinny_static: problem exceeds the static scratch: ", detail);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e = cudaMemsetAsync(d->tickets, 0, sizeof(int) * tiles, stream);
  if (e != cudaSuccess) return static_fail(HB_ERR_CUDA, "skinny_static: cudaMemsetAsync: ", cudaGetErrorString(e));
  hb_gemm_args a;
  memset(&a, 0, sizeof(a));
  a.A = A; a.B = B; a.C = C;
  a.M = M; a.N = N; a.K = K;
  a.lda = K; a.ldb = K; a.ldc = N;
  st = hb_launch_gemm_skinny_raw(nullptr, stream, a, d->partial, d->tickets, grid, max_seg, tiles, 0, d->status);
  if (st != HB_OK) return static_fail(st, "skinny_static: launch failed (descriptor encoding or kernel launch)");
  return HB_OK;
}

// Copies the static status words back (blocking): out[0] != 0 means a bounded wait inside
// a static launch on `device` gave up since the last call.  Clears them.
extern "C" hb_status hb_static_status(int32_t device, int32_t* out4) {
  if (!out4) return HB_ERR_INVALID;
  StaticDev* d = nullptr;
  hb_status st = static_setup(device, &d);
  if (st != HB_OK) return st;
  cudaError_t e = cudaMemcpy(out4, d->status, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && out4[0] != 0) e = cudaMemset(d->status, 0, 4 * sizeof(int32_t));
  return e == cudaSuccess ? HB_OK : static_fail(HB_ERR_CUDA, "skinny_static: status copy: ", cudaGetErrorString(e));
}
