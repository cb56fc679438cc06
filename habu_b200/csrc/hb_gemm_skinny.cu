// Skinny (decode-shaped) bf16 GEMM for sm_100a: C[M,N] = A[M,K] . B[K,N] with M <= 64.
// The product is HBM-bound on reading B (N*K*2 bytes), so the kernel is built to keep
// every SM streaming B:
//   * operands are swapped: a 128-row slab of B (stored [N,K], K contiguous) is the MMA's
//     M-side operand and A (padded to a multiple of 16 rows by TMA zero fill) is its N-side
//     operand, so tcgen05.mma runs at M=128, N=16..64 and no tensor-core work is wasted on
//     padding M up to 128;
//   * K is split into `split` slices so that tiles * split CTAs cover the machine (two
//     CTAs fit per SM); each CTA pipelines its slice through a TMA ring;
//   * every CTA writes its fp32 partial tile to scratch; the last CTA to finish a tile
//     (atomic ticket) adds the partials in slice order -- a fixed order, so the result is
//     bit-identical run to run -- rounds to bf16 once and writes C.
// Scratch: split * N * Mpad floats of partials plus one ticket per tile (tickets are left
// at zero by the CTA that consumes them).
// Algorithmic traffic per launch: (N*K + M*K + M*N) * 2 bytes.
#include <stdlib.h>
#include <string.h>

#include "hb_internal.h"
#include "hb_ptx.cuh"

namespace {

using namespace hb;

constexpr int BN_ROWS = 128;   // rows of B per tile (MMA M)
constexpr int BK = 64;
constexpr int STAGES = 4;     // 4 x 24 KB: two CTAs fit in one SM's shared memory
constexpr int SK_THREADS = 192;
constexpr int MAX_MPAD = 64;

struct SkinnyParams {
  __nv_bfloat16* C;
  float* partial;      // [split][N_tiles*128][mpad]
  int* tickets;        // [N_tiles]
  int M, N, K;
  int64_t ldc;
  int mpad;            // M rounded up to 16
  int split;
  int kb_per_split;    // k-blocks per slice
  int32_t* status;
};

struct SkSmem {
  static constexpr int B_BYTES = BN_ROWS * BK * 2;       // 16 KB
  static constexpr int A_BYTES = MAX_MPAD * BK * 2;      // 8 KB (mpad rows used)
  static constexpr int OFF_B = 0;
  static constexpr int OFF_A = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_BAR = OFF_A + STAGES * A_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 1;
  static constexpr int OFF_TMEM_PTR = OFF_BAR + NUM_BARS * 8;
  static constexpr int OFF_ABORT = OFF_TMEM_PTR + 4;
  static constexpr int OFF_LAST = OFF_ABORT + 4;
  static constexpr int TOTAL = OFF_LAST + 4;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

__global__ void __launch_bounds__(SK_THREADS, 2)
hb_gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmA,
                      const SkinnyParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sB = smem_base + SkSmem::OFF_B;
  const uint32_t sA = smem_base + SkSmem::OFF_A;
  const uint32_t bar_full = smem_base + SkSmem::OFF_BAR;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_done = bar_empty + STAGES * 8;
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + SkSmem::OFF_TMEM_PTR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SkSmem::OFF_ABORT);
  volatile int* is_last = reinterpret_cast<volatile int*>(smem + SkSmem::OFF_LAST);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile = blockIdx.x / p.split;
  const int slice = blockIdx.x % p.split;
  const int n0 = tile * BN_ROWS;
  const int num_kb_total = (p.K + BK - 1) / BK;
  const int kb0 = slice * p.kb_per_split;
  const int kb1 = min(num_kb_total, kb0 + p.kb_per_split);
  const int num_kb = max(0, kb1 - kb0);
  constexpr uint32_t TMEM_COLS = 64;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *is_last = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    mbar_init(bar_done, 1);
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
  const uint32_t a_bytes = static_cast<uint32_t>(p.mpad) * BK * 2;

  if (warp == 0) {
    if (elect_one()) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(bar_empty + s * 8, phase ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(bar_full + s * 8, SkSmem::B_BYTES + a_bytes);
        tma_load_2d(sB + s * SkSmem::B_BYTES, &tmB, bar_full + s * 8, kb * BK, n0);
        tma_load_2d(sA + s * SkSmem::A_BYTES, &tmA, bar_full + s * 8, kb * BK, 0);
        if (++s == STAGES) { s = 0; phase ^= 1; }
      }
      if (!ok && p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_SPLITK; p.status[2] = 1; }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_bf16(BN_ROWS, p.mpad, 0, 0);
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(bar_full + s * 8, phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_ss<1>(tmem_base, umma_desc_k_sw128(sB + s * SkSmem::B_BYTES + k * 32),
                     umma_desc_k_sw128(sA + s * SkSmem::A_BYTES + k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit<1>(bar_empty + s * 8);
        if (++s == STAGES) { s = 0; phase ^= 1; }
      }
      if (ok) umma_commit<1>(bar_done);
      if (!ok && p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_SPLITK; p.status[2] = 2; }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int q = warp & 3;
    const int r = q * 32 + lane;                 // row of the B slab = output column n0 + r
    const int etid = (warp - 2) * 32 + lane;     // 0..127
    bool ok = true;
    if (num_kb > 0) ok = mbar_wait(bar_done, 0, abort_flag);
    float acc[MAX_MPAD];
#pragma unroll
    for (int i = 0; i < MAX_MPAD; ++i) acc[i] = 0.f;
    if (ok && num_kb > 0) {
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
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
    }
    const int64_t n_rows_padded = static_cast<int64_t>(gridDim.x / p.split) * BN_ROWS;
    float* mine = p.partial + (static_cast<int64_t>(slice) * n_rows_padded + n0 + r) * p.mpad;
    if (p.split > 1) {
#pragma unroll
      for (int c = 0; c < MAX_MPAD / 4; ++c)
        if (c * 4 < p.mpad)
          *reinterpret_cast<float4*>(mine + c * 4) = make_float4(acc[c * 4], acc[c * 4 + 1], acc[c * 4 + 2], acc[c * 4 + 3]);
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (etid == 0) {
        const int ticket = atomicAdd(p.tickets + tile, 1);
        const int last = ticket == p.split - 1;
        if (last) p.tickets[tile] = 0;           // leave the ticket ready for the next launch
        *is_last = last;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*is_last) {
        __threadfence();
#pragma unroll
        for (int i = 0; i < MAX_MPAD; ++i) acc[i] = 0.f;
        for (int s = 0; s < p.split; ++s) {      // fixed order: bit-identical run to run
          const float* src = p.partial + (static_cast<int64_t>(s) * n_rows_padded + n0 + r) * p.mpad;
#pragma unroll
          for (int c = 0; c < MAX_MPAD / 4; ++c)
            if (c * 4 < p.mpad) {
              const float4 v = __ldcg(reinterpret_cast<const float4*>(src + c * 4));
              acc[c * 4] += v.x; acc[c * 4 + 1] += v.y; acc[c * 4 + 2] += v.z; acc[c * 4 + 3] += v.w;
            }
        }
      }
    }
    if ((p.split == 1 || *is_last) && ok) {
      const int n = n0 + r;
      if (n < p.N) {
#pragma unroll
        for (int m = 0; m < MAX_MPAD; ++m)
          if (m < p.M) p.C[static_cast<int64_t>(m) * p.ldc + n] = __float2bfloat16_rn(acc[m]);
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

}  // namespace

bool hb_gemm_skinny_applicable(const hb_gemm_args& a) {
  return a.M <= MAX_MPAD && !a.a_mn_major && !a.b_mn_major && a.epilogue == HB_EPI_NONE && a.N >= 256;
}

// Chooses the K split and reports the scratch the launch needs.
void hb_gemm_skinny_plan(int sm_count, int64_t M, int64_t N, int64_t K, int* split, int* kb_per_split,
                         size_t* partial_floats, int* tiles) {
  const int t = (int)((N + BN_ROWS - 1) / BN_ROWS);
  const int num_kb = (int)((K + BK - 1) / BK);
  const int mpad = (int)((M + 15) / 16) * 16;
  int s = (2 * sm_count) / t;                  // one wave of two CTAs per SM
  if (const char* e = getenv("HB_SKINNY_SPLIT")) s = atoi(e);
  int max_s = num_kb / 8 > 0 ? num_kb / 8 : 1; // at least 8 k-blocks per slice
  if (s > max_s) s = max_s;
  if (s > 16) s = 16;
  if (s < 1) s = 1;
  int per = (num_kb + s - 1) / s;
  s = (num_kb + per - 1) / per;                // drop empty slices
  *split = s;
  *kb_per_split = per;
  *tiles = t;
  *partial_floats = s > 1 ? (size_t)s * t * BN_ROWS * mpad : 0;
}

hb_status hb_launch_gemm_skinny_raw(hb_ctx* ctx, cudaStream_t stream, const hb_gemm_args& a, float* partial, int* tickets,
                                    int split, int kb_per_split, int tiles, int32_t* status) {
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
  p.split = split;
  p.kb_per_split = kb_per_split;
  p.status = status;
  // the attribute is per device: one flag for each device this process launches on
  static bool attr_set_dev[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  bool& attr_set = attr_set_dev[dev & 63];
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(hb_gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SkSmem::DYN_BYTES);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaFuncSetAttribute(skinny gemm)");
    attr_set = true;
  }
  hb_gemm_skinny_kernel<<<tiles * split, SK_THREADS, SkSmem::DYN_BYTES, stream>>>(tmB, tmA, p);
  return hb_check_cuda(ctx, cudaGetLastError(), "skinny gemm launch");
}

hb_status hb_launch_gemm_skinny(hb_ctx* ctx, const hb_gemm_args& a) {
  int split, per, tiles;
  size_t floats;
  hb_gemm_skinny_plan(ctx->sm_count, a.M, a.N, a.K, &split, &per, &floats, &tiles);
  if (tiles > HB_MAX_SPLITK_TILES) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "matmul: N too large for the split-K path");
  void* ws = nullptr;
  if (floats) {
    hb_status st = hb_get_scratch(ctx, HB_SCRATCH_WORKSPACE, floats * sizeof(float), &ws);
    if (st != HB_OK) return st;
  }
  hb_status st = hb_launch_gemm_skinny_raw(ctx, ctx->stream, a, static_cast<float*>(ws), ctx->d_tickets, split, per, tiles,
                                           ctx->d_status);
  if (st == HB_OK) ctx->launches++;
  return st;
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
// Limits: partials split * ceil(N/128)*128 * Mpad <= HB_STATIC_MAX_PARTIAL_FLOATS and
// ceil(N/128) <= HB_STATIC_MAX_TILES; larger problems are refused with HB_ERR_UNSUPPORTED.
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
hb_status static_setup(int device, StaticDev** out) {
  if (device < 0 || device >= 64) return static_fail(HB_ERR_INVALID, "skinny_static: device index out of range");
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
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess || cur != device)
    return static_fail(HB_ERR_INVALID, "skinny_static: `device` must be the current CUDA device of the calling thread");
  StaticDev* d = nullptr;
  hb_status st = static_setup(device, &d);
  if (st != HB_OK) return st;
  int split, per, tiles;
  size_t floats;
  hb_gemm_skinny_plan(d->sm_count, M, N, K, &split, &per, &floats, &tiles);
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
  st = hb_launch_gemm_skinny_raw(nullptr, stream, a, d->partial, d->tickets, split, per, tiles, d->status);
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
