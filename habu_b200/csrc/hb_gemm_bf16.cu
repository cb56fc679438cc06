// bf16 GEMM for sm_100a: C[M,N] = epilogue(A[M,K] . B[K,N]), fp32 accumulation in tensor
// memory, bf16 output.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of A (128 x 64) and B (BN x 64)
//               tiles, 128-byte swizzled, into a STAGES-deep shared-memory ring;
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) four
//               times per 64-wide k-block, tcgen05.commit releases the ring slot, and a
//               final commit per tile publishes the accumulator;
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one TMEM lane = one output row per
//               thread), apply the epilogue, round to bf16 once, 16-byte global stores.
// Two accumulators (2 x BN TMEM columns) let the epilogue of tile i overlap the mainloop
// of tile i+1.  Operands may be K-major (K contiguous) or MN-major; both are described to
// the tensor core by shared-memory descriptors over the layout TMA writes.
//
// Algorithmic traffic per launch: (M*K + N*K + M*N) * 2 bytes; work 2*M*N*K flop.
#include <stdio.h>
#include <stdlib.h>

#include "hb_internal.h"
#include "hb_ptx.cuh"

namespace {

using namespace hb;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  __nv_bfloat16* C;
  const __nv_bfloat16* R;   // residual (or null)
  int M, N, K;
  int64_t ldc, ldr;
  int tiles_m, tiles_n;
  int raster_group;         // tiles_m grouped per sweep over N (L2 reuse)
  int epilogue;
  int a_mn, b_mn;           // operand is MN-major
  int32_t* status;
  // A's rows arrive while the kernel runs (the gathered output of a fused collective): the
  // producer waits for the "rows ready" word of a row block before its first load from it.
  const uint32_t* ready;    // null: A is complete at launch
  uint32_t ready_epoch;     // a word is set when (int32)(word - ready_epoch) >= 0
  uint32_t ready_spin;      // polls before the wait gives up
  int ready_rows;           // rows per word
  int perm_world, perm_rank;  // > 1: M-tiles are visited owner by owner in turn, this rank's rows first
  int tma_store;            // the epilogue stages 32 x 32 blocks in shared memory and stores them with TMA
};

// Output staging: each of the four epilogue warps owns two buffers of 32 rows x 32 bf16 columns
// (64-byte rows, 64-byte swizzle: the 16-byte piece c of row r sits at piece c ^ ((r >> 1) & 3),
// so that the row-per-lane writes of a warp spread over all banks).
constexpr int STAGE_BUF_BYTES = 32 * 64;
constexpr int STAGE_BYTES = 4 * 2 * STAGE_BUF_BYTES;

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Waits until rows [m0, m0 + nrows) of A have been published.  `seen` caches the last block
// found ready (tiles of one M-tile follow each other).  The rows were written by other GPUs
// (or through the switch) with generic stores; the loads that follow go through the async
// proxy, hence the proxy fence after the acquire.
__device__ __forceinline__ bool wait_rows_ready(const GemmParams& p, int m0, int nrows, int& seen, volatile int* abort_flag) {
  const int last_row = min(m0 + nrows, p.M) - 1;
  if (last_row < m0) return true;
  const int b0 = m0 / p.ready_rows, b1 = last_row / p.ready_rows;
  bool polled = false;
  for (int b = b0; b <= b1; ++b) {
    if (b == seen) continue;
    uint32_t it = 0;
    while (static_cast<int32_t>(ld_acquire_sys_u32(p.ready + b) - p.ready_epoch) < 0) {
      if (++it > p.ready_spin || ((it & 255u) == 0 && *abort_flag)) { *abort_flag = 1; return false; }
      __nanosleep(100);
    }
    seen = b;
    polled = true;
  }
  if (polled) asm volatile("fence.proxy.async.global;" ::: "memory");
  return true;
}

// A ring stage holds KPS consecutive 64-wide k-blocks of both operands (KPS = 2: a 128-wide
// K step per barrier round trip, half as many producer/consumer hand-offs).
template <int BN, int STAGES, int KPS>
struct SmemLayout {
  static constexpr int A_BLOCK = BM * BK * 2;
  static constexpr int B_BLOCK = BN * BK * 2;
  static constexpr int A_BYTES = KPS * A_BLOCK;
  static constexpr int B_BYTES = KPS * B_BLOCK;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_BAR = OFF_B + STAGES * B_BYTES;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int OFF_TMEM_PTR = OFF_BAR + NUM_BARS * 8;
  static constexpr int OFF_ABORT = OFF_TMEM_PTR + 4;
  static constexpr int OFF_STAGE = (OFF_ABORT + 4 + 1023) & ~1023;   // output staging of the epilogue warps
  static constexpr int TOTAL = OFF_STAGE + STAGE_BYTES;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack for 1024-byte alignment
};

__device__ __forceinline__ void tile_coords(int tile, const GemmParams& p, int& tm, int& tn) {
  // Sweep N inside groups of `raster_group` M-tiles so that concurrently resident CTAs
  // share A rows and B columns in L2.
  const int g = p.raster_group;
  const int per_group = g * p.tiles_n;
  const int group = tile / per_group;
  const int first_m = group * g;
  const int rows = min(g, p.tiles_m - first_m);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
  if (p.perm_world > 1) {
    // visiting index -> M-tile: owners in turn (this rank first), block by block within an owner
    const int per_owner = p.tiles_m / p.perm_world;
    const int owner = (tm % p.perm_world + p.perm_rank) % p.perm_world;
    tm = owner * per_owner + tm / p.perm_world;
  }
}

__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

// SwiGLU of one 32-column accumulator chunk: columns interleave (gate, up), 16 outputs
// out[j] = silu(acc[2j]) * acc[2j+1], packed in pairs.
__device__ __forceinline__ void swiglu_chunk(const uint32_t (&v)[32], uint32_t (&o)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float g0 = __uint_as_float(v[4 * j]), u0 = __uint_as_float(v[4 * j + 1]);
    const float g1 = __uint_as_float(v[4 * j + 2]), u1 = __uint_as_float(v[4 * j + 3]);
    o[j] = pack_bf16x2(silu(g0) * u0, silu(g1) * u1);
  }
}

// The other epilogues of one 32-column chunk of row `row` (none, GELU, + residual), in fp32.
__device__ __forceinline__ void epilogue_values(const GemmParams& p, int row, int col0, const uint32_t (&v)[32],
                                                float (&f)[32]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
  if (p.epilogue == HB_EPI_GELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = gelu_erf(f[j]);
  } else if (p.epilogue == HB_EPI_RESIDUAL && row < p.M) {
    const __nv_bfloat16* r = p.R + static_cast<int64_t>(row) * p.ldr + col0;
    if (((p.ldr & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.R) & 15) == 0) && col0 + 32 <= p.N) {
#pragma unroll
      for (int j4 = 0; j4 < 4; ++j4) {
        const uint4 rv = __ldg(reinterpret_cast<const uint4*>(r) + j4);
        const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 rf = __bfloat1622float2(r2[j]);
          f[j4 * 8 + 2 * j] += rf.x;
          f[j4 * 8 + 2 * j + 1] += rf.y;
        }
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) f[j] += __bfloat162float(r[j]);
    }
  }
}

// One 32-column chunk of one output row: apply the epilogue, round to bf16 once, store.
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, bool vec_ok, int row, int col0,
                                               const uint32_t (&v)[32]) {
  if (row >= p.M || col0 >= p.N) return;
    if (p.epilogue == HB_EPI_SWIGLU) {
      // columns interleave (gate, up): out[j] = silu(acc[2j]) * acc[2j+1]
      const int ocol0 = col0 >> 1;
      const int on = p.N >> 1;
      __nv_bfloat16* dst = p.C + static_cast<int64_t>(row) * p.ldc + ocol0;
      uint32_t o[8];
      swiglu_chunk(v, o);
      if (vec_ok && ocol0 + 16 <= on) {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        d4[0] = make_uint4(o[0], o[1], o[2], o[3]);
        d4[1] = make_uint4(o[4], o[5], o[6], o[7]);
      } else {
        const __nv_bfloat16* ob = reinterpret_cast<const __nv_bfloat16*>(o);
        for (int j = 0; j < 16; ++j)
          if (ocol0 + j < on) dst[j] = ob[j];
      }
    } else {
      float f[32];
      epilogue_values(p, row, col0, v, f);
      uint32_t o[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) o[j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
      __nv_bfloat16* dst = p.C + static_cast<int64_t>(row) * p.ldc + col0;
      if (vec_ok && col0 + 32 <= p.N) {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          d4[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
      } else {
        const __nv_bfloat16* ob = reinterpret_cast<const __nv_bfloat16*>(o);
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) dst[j] = ob[j];
      }
    }
}

// The same 32-column chunk through shared memory: every lane applies the epilogue to its row
// and writes the 64 bytes into the warp's staging buffer; lane 0 then hands the 32 x 32 block
// to TMA, which writes full lines (a warp's own stores touch 32 different rows with 16 bytes
// each) and clips the block at the matrix edge.  `row0` is the first of the warp's 32 rows, `c`
// the running number of the chunk over all tiles of this warp (a tile has an even number of
// chunks), `stage` the warp's two buffers, used in turn.  With the SwiGLU epilogue a chunk yields
// 16 output columns, so two consecutive chunks fill one block.
__device__ __forceinline__ void epilogue_chunk_staged(const GemmParams& p, const CUtensorMap* tmC, uint32_t stage,
                                                      int lane, int row0, int col0, int c, const uint32_t (&v)[32]) {
  if (p.epilogue == HB_EPI_SWIGLU) {
    stage += ((c >> 1) & 1) * STAGE_BUF_BYTES;
    const int odd = c & 1;
    if (!odd) {
      if (lane == 0) tma_store_wait_read<1>();
      __syncwarp();
    }
    if (row0 < p.M && col0 < p.N) {
      const uint32_t mine = stage + lane * 64;
      const int sw = (lane >> 1) & 3;
      uint32_t o[8];
      swiglu_chunk(v, o);
#pragma unroll
      for (int h = 0; h < 2; ++h)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(mine + (((odd * 2 + h) ^ sw) << 4)),
                     "r"(o[4 * h]), "r"(o[4 * h + 1]), "r"(o[4 * h + 2]), "r"(o[4 * h + 3])
                     : "memory");
    }
    if (odd) {
      if (row0 < p.M && col0 - 32 < p.N) {     // the pair's first chunk was inside the matrix
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) tma_store_2d(tmC, stage, (col0 - 32) >> 1, row0);
      }
      if (lane == 0) tma_store_commit();
    }
    return;
  }
  stage += (c & 1) * STAGE_BUF_BYTES;
  if (lane == 0) tma_store_wait_read<1>();     // the store issued two chunks ago has read this buffer
  __syncwarp();
  if (row0 < p.M && col0 < p.N) {
    float f[32];
    epilogue_values(p, row0 + lane, col0, v, f);
    const uint32_t mine = stage + lane * 64;
    const int sw = (lane >> 1) & 3;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t o0 = pack_bf16x2(f[8 * c], f[8 * c + 1]), o1 = pack_bf16x2(f[8 * c + 2], f[8 * c + 3]);
      const uint32_t o2 = pack_bf16x2(f[8 * c + 4], f[8 * c + 5]), o3 = pack_bf16x2(f[8 * c + 6], f[8 * c + 7]);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(mine + ((c ^ sw) << 4)), "r"(o0), "r"(o1),
                   "r"(o2), "r"(o3)
                   : "memory");
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) tma_store_2d(tmC, stage, col0, row0);
  }
  if (lane == 0) tma_store_commit();           // one group per chunk, empty or not: keeps the count uniform
}

template <int BN, int STAGES, int KPS>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
hb_gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using L = SmemLayout<BN, STAGES, KPS>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t sA = smem_base + L::OFF_A;
  const uint32_t sB = smem_base + L::OFF_B;
  const uint32_t bar_full = smem_base + L::OFF_BAR;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_tfull = bar_empty + STAGES * 8;
  const uint32_t bar_tempty = bar_tfull + 2 * 8;
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::OFF_TMEM_PTR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::OFF_ABORT);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128
                                 : (2 * BN <= 256) ? 256 : 512;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
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

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + BK * KPS - 1) / (BK * KPS);   // ring steps per tile; a block past K loads zeros

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      int seen = -1;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, p, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        if (p.ready && !wait_rows_ready(p, m0, BM, seen, abort_flag)) {
          if (p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_GEMM; p.status[2] = 4; }
          break;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + s * 8, phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(bar_full + s * 8, L::A_BYTES + L::B_BYTES);
#pragma unroll
          for (int kk = 0; kk < KPS; ++kk) {
            const int k0 = (kb * KPS + kk) * BK;
            const uint32_t a_dst = sA + s * L::A_BYTES + kk * L::A_BLOCK;
            const uint32_t b_dst = sB + s * L::B_BYTES + kk * L::B_BLOCK;
            if (!p.a_mn) {
              tma_load_2d(a_dst, &tmA, bar_full + s * 8, k0, m0);
            } else {
              // M-major A: two boxes of 64 (M) x 64 (K); box c holds rows m0+64c..+63
              tma_load_2d(a_dst, &tmA, bar_full + s * 8, m0, k0);
              tma_load_2d(a_dst + L::A_BLOCK / 2, &tmA, bar_full + s * 8, m0 + 64, k0);
            }
            if (!p.b_mn) {
              tma_load_2d(b_dst, &tmB, bar_full + s * 8, k0, n0);
            } else {
#pragma unroll
              for (int c = 0; c < BN / 64; ++c)
                tma_load_2d(b_dst + c * (64 * BK * 2), &tmB, bar_full + s * 8, n0 + 64 * c, k0);
            }
          }
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
      if (!ok && p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_GEMM; p.status[2] = 1; }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_bf16(BM, BN, p.a_mn, p.b_mn);
      int s = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(bar_tempty + acc * 8, acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_full + s * 8, phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < KPS; ++kk) {
            const uint32_t a_addr = sA + s * L::A_BYTES + kk * L::A_BLOCK;
            const uint32_t b_addr = sB + s * L::B_BYTES + kk * L::B_BLOCK;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // K-major: 16 bf16 = 32 bytes further along the 128-byte swizzled row.
              // MN-major: 16 k-rows = two 8-row groups of 1024 bytes further.
              const uint64_t ad = p.a_mn ? umma_desc_mn_sw128(a_addr + k * 2048, L::A_BLOCK / 2, 1024)
                                         : umma_desc_k_sw128(a_addr + k * 32);
              const uint64_t bd = p.b_mn ? umma_desc_mn_sw128(b_addr + k * 2048, 64 * BK * 2, 1024)
                                         : umma_desc_k_sw128(b_addr + k * 32);
              umma_ss<1>(d_tmem, ad, bd, idesc, (kb | kk | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit<1>(bar_empty + s * 8);
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (ok) umma_commit<1>(bar_tfull + acc * 8);
      }
      if (!ok && p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_GEMM; p.status[2] = 2; }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;               // TMEM lane quarter this warp may access
    const int row_in_tile = q * 32 + lane;
    int it = 0;
    bool ok = true;
    const bool vec_ok = ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const uint32_t stage_mine = smem_base + L::OFF_STAGE + q * 2 * STAGE_BUF_BYTES;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      int tm, tn;
      tile_coords(tile, p, tm, tn);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(bar_tfull + acc * 8, acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + row_in_tile;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_row + c * 32, v);
        tmem_wait_ld();
        const int col0 = tn * BN + c * 32;
        if (p.tma_store)
          epilogue_chunk_staged(p, &tmC, stage_mine, lane, tm * BM + q * 32, col0, it * (BN / 32) + c, v);
        else
          epilogue_chunk(p, vec_ok, row, col0, v);
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + acc * 8);
    }
    if (p.tma_store && lane == 0) tma_store_wait<0>();   // the staged blocks have left shared memory and landed
    if (!ok && p.status && lane == 0) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_GEMM; p.status[2] = 3; }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster (the two SMs of a TPC) share one 256 x 256 tile.
// Each CTA loads its own 128 rows of A and its own 128 of the tile's 256 B rows; the
// leader CTA issues tcgen05.mma.cta_group::2 (M = 256, N = 256), which reads A from each
// CTA's shared memory and the two B halves from both, and leaves rows 0..127 of the tile
// in the leader's tensor memory and rows 128..255 in the peer's.  Per k-block a CTA moves
// 32 KB instead of 48 KB, so six stages fit and L2 -> SM traffic drops by a third.
// The arrivals a CTA makes on its partner's barriers use the default (CTA-scope) release:
// with an explicit cluster-scope release on each of them the kernel ran at half speed.
// Measured: 8192^3 in 0.708 ms (1553 TFLOP/s) against 0.763 ms for the one-CTA kernel.
//   full[s]    leader only, 2 arrivals (+ 64 KB of TMA bytes from both CTAs)
//   empty[s]   one per CTA, signalled by the leader's commit in both CTAs
//   tfull[a]   one per CTA, same way;   tempty[a]  leader only, 256 arrivals (both epilogues)
// No load is multicast: each CTA fetches exactly the bytes it owns.
// ------------------------------------------------------------------------------------
// BN2 is the width of the pair's tile (256 x BN2, BN2 = 256 or 128): each CTA holds 128 rows of
// A and BN2 / 2 rows of B per k-block.  The narrower tile gives three times as many tiles on
// short-N products (a 768-wide QKV shard), where 256 x 256 tiles leave a third of the last wave
// empty.
template <int BN2, int STAGES, int KPS>
struct SmemLayout2 {
  static constexpr int A_BLOCK = 128 * BK * 2;
  static constexpr int B_BLOCK = (BN2 / 2) * BK * 2;
  static constexpr int A_BYTES = KPS * A_BLOCK;
  static constexpr int B_BYTES = KPS * B_BLOCK;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_BAR = OFF_B + STAGES * B_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int OFF_TMEM_PTR = OFF_BAR + NUM_BARS * 8;
  static constexpr int OFF_ABORT = OFF_TMEM_PTR + 4;
  static constexpr int OFF_STAGE = (OFF_ABORT + 4 + 1023) & ~1023;
  static constexpr int TOTAL = OFF_STAGE + STAGE_BYTES;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

template <int BN2, int STAGES, int KPS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
hb_gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using L = SmemLayout2<BN2, STAGES, KPS>;
  constexpr uint32_t TMEM_COLS = 2 * BN2;          // two accumulators: 512 or 256 columns
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sA = smem_base + L::OFF_A;
  const uint32_t sB = smem_base + L::OFF_B;
  const uint32_t bar_full = smem_base + L::OFF_BAR;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_tfull = bar_empty + STAGES * 8;
  const uint32_t bar_tempty = bar_tfull + 2 * 8;
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::OFF_TMEM_PTR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::OFF_ABORT);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + s * 8, 2);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + a * 8, 1);
      mbar_init(bar_tempty + a * 8, 256);
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {   // the same warp in both CTAs, same destination address
    tmem_alloc<2>(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), TMEM_COLS);
    tmem_relinquish<2>();
  }
  tc_fence_before();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int num_tiles = p.tiles_m * p.tiles_n;     // 256 x BN2 tiles
  const int num_kb = (p.K + BK * KPS - 1) / (BK * KPS);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      int seen = -1;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        tile_coords(tile, p, tm, tn);
        const int m0 = tm * 256 + static_cast<int>(cta_rank) * 128;
        const int n0 = tn * BN2 + static_cast<int>(cta_rank) * (BN2 / 2);
        if (p.ready && !wait_rows_ready(p, m0, 128, seen, abort_flag)) {
          if (p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_GEMM; p.status[2] = 14; }
          break;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + s * 8, phase ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t full_leader = mapa(bar_full + s * 8, 0);
          if (leader) mbar_arrive_expect_tx(bar_full + s * 8, L::A_BYTES + L::B_BYTES);
          else mbar_arrive_expect_tx_cluster(full_leader, L::A_BYTES + L::B_BYTES);
#pragma unroll
          for (int kk = 0; kk < KPS; ++kk) {
            const int k0 = (kb * KPS + kk) * BK;
            const uint32_t a_dst = sA + s * L::A_BYTES + kk * L::A_BLOCK;
            const uint32_t b_dst = sB + s * L::B_BYTES + kk * L::B_BLOCK;
            if (!p.a_mn) {
              tma_load_2d_pair(a_dst, &tmA, full_leader, k0, m0);
            } else {   // M-major A: two boxes of 64 (M) x 64 (K)
              tma_load_2d_pair(a_dst, &tmA, full_leader, m0, k0);
              tma_load_2d_pair(a_dst + L::A_BLOCK / 2, &tmA, full_leader, m0 + 64, k0);
            }
            if (!p.b_mn) {
              tma_load_2d_pair(b_dst, &tmB, full_leader, k0, n0);
            } else {   // N-major B: boxes of 64 (N) x 64 (K)
#pragma unroll
              for (int c = 0; c < BN2 / 128; ++c)
                tma_load_2d_pair(b_dst + c * (64 * BK * 2), &tmB, full_leader, n0 + 64 * c, k0);
            }
          }
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
      if (!ok && p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_GEMM; p.status[2] = 11; }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && elect_one()) {
      const uint32_t idesc = umma_idesc_bf16(256, BN2, p.a_mn, p.b_mn);
      int s = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(bar_tempty + acc * 8, acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN2;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_full + s * 8, phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < KPS; ++kk) {
            const uint32_t a_addr = sA + s * L::A_BYTES + kk * L::A_BLOCK, b_addr = sB + s * L::B_BYTES + kk * L::B_BLOCK;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t ad = p.a_mn ? umma_desc_mn_sw128(a_addr + k * 2048, L::A_BLOCK / 2, 1024)
                                         : umma_desc_k_sw128(a_addr + k * 32);
              const uint64_t bd = p.b_mn ? umma_desc_mn_sw128(b_addr + k * 2048, 64 * BK * 2, 1024)
                                         : umma_desc_k_sw128(b_addr + k * 32);
              umma_ss<2>(d_tmem, ad, bd, idesc, (kb | kk | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit_pair_mcast(bar_empty + s * 8, 3);      // frees the slot in both CTAs
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair_mcast(bar_tfull + acc * 8, 3);
      }
      if (!ok && p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_GEMM; p.status[2] = 12; }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    int it = 0;
    bool ok = true;
    const bool vec_ok = ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const uint32_t tempty_leader = mapa(bar_tempty, 0);
    const uint32_t stage_mine = smem_base + L::OFF_STAGE + q * 2 * STAGE_BUF_BYTES;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
      int tm, tn;
      tile_coords(tile, p, tm, tn);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(bar_tfull + acc * 8, acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * 256 + static_cast<int>(cta_rank) * 128 + row_in_tile;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN2;
#pragma unroll 1
      for (int c = 0; c < BN2 / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_row + c * 32, v);
        tmem_wait_ld();
        if (p.tma_store)
          epilogue_chunk_staged(p, &tmC, stage_mine, lane, tm * 256 + static_cast<int>(cta_rank) * 128 + q * 32,
                                tn * BN2 + c * 32, it * (BN2 / 32) + c, v);
        else
          epilogue_chunk(p, vec_ok, row, tn * BN2 + c * 32, v);
      }
      tc_fence_before();
      mbar_arrive_cluster(tempty_leader + acc * 8);
    }
    if (p.tma_store && lane == 0) tma_store_wait<0>();
    if (!ok && p.status && lane == 0) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_GEMM; p.status[2] = 13; }
  }

  // Neither CTA may leave while its partner can still signal its barriers or read its
  // shared memory.
  tc_fence_before();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<2>(tmem_base, TMEM_COLS);
  }
}

struct GemmVariant {
  int cluster;      // 1: one CTA per 128 x bn tile; 2: CTA pair per 256 x bn tile
  int bn;           // tile N
  int stages;       // ring depth
  int kps;          // 64-wide k-blocks per ring stage (tile K = 64 * kps)
};
// Every kernel instantiation in the library (bytes per stage = kps * 128 * (128 + bn) for one
// CTA, kps * 128 * (128 + bn / 2) per CTA of a pair).  No ring exceeds 192 KB: a seven-stage
// 256 x 256 pair ring (224 KB) measured within 0.5 % of the six-stage one, and it leaves no
// shared memory for a collective kernel's CTA on the same SM, which is what the overlapped
// schedules of the tensor-parallel block rely on.
constexpr GemmVariant kVariants[] = {
    {1, 256, 4, 1}, {1, 256, 3, 1}, {1, 256, 2, 2},
    {1, 128, 6, 1}, {1, 128, 4, 1}, {1, 128, 3, 2},
    {1, 64, 8, 1},  {1, 64, 5, 1},  {1, 64, 4, 2},
    {2, 256, 6, 1}, {2, 256, 5, 1}, {2, 256, 4, 1}, {2, 256, 3, 2},
    {2, 128, 8, 1}, {2, 128, 6, 1}, {2, 128, 4, 2},
};
constexpr int kRasters[] = {8, 16, 4, 2};        // M-tiles per sweep over N
constexpr int kNumVariants = sizeof(kVariants) / sizeof(kVariants[0]);
constexpr int kNumRasters = sizeof(kRasters) / sizeof(kRasters[0]);
constexpr int kNumConfigs = kNumVariants * kNumRasters;   // config_id = variant * kNumRasters + raster index

template <int BN, int STAGES, int KPS>
hb_status launch_cfg(hb_ctx* ctx, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, GemmParams& p) {
  using L = SmemLayout<BN, STAGES, KPS>;
  static_assert(L::DYN_BYTES <= 227 * 1024, "ring does not fit shared memory");
  auto kern = hb_gemm_bf16_kernel<BN, STAGES, KPS>;
  static bool attr_set[64] = {};
  if (!attr_set[ctx->device & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         L::DYN_BYTES);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaFuncSetAttribute(gemm)");
    attr_set[ctx->device & 63] = true;
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
  kern<<<grid, GEMM_THREADS, L::DYN_BYTES, ctx->stream>>>(tmA, tmB, tmC, p);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "gemm launch");
}

template <int BN2, int STAGES, int KPS>
hb_status launch_pair(hb_ctx* ctx, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, GemmParams& p) {
  using L = SmemLayout2<BN2, STAGES, KPS>;
  static_assert(L::DYN_BYTES <= 227 * 1024, "ring does not fit shared memory");
  auto kern = hb_gemm_bf16_pair_kernel<BN2, STAGES, KPS>;
  // The grid is capped by the number of clusters that can be resident at once (the occupancy
  // query's answer: not every SM has a pairable neighbour, so this is below sm_count / 2).
  static int resident_pairs[64] = {};
  if (!resident_pairs[ctx->device & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaFuncSetAttribute(pair gemm)");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctx->sm_count & ~1u);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = L::DYN_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess || n < 1) { cudaGetLastError(); n = ctx->sm_count / 2 - 8; }
    if (getenv("HB_DEBUG")) fprintf(stderr, "[habu_b200] pair gemm: %d resident clusters (query status %d)\n", n, (int)e);
    resident_pairs[ctx->device & 63] = n;
  }
  p.tiles_m = (p.M + 255) / 256;
  p.tiles_n = (p.N + BN2 - 1) / BN2;
  const int tiles = p.tiles_m * p.tiles_n;
  const int max_pairs = resident_pairs[ctx->device & 63];
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, GEMM_THREADS, L::DYN_BYTES, ctx->stream>>>(tmA, tmB, tmC, p);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "pair gemm launch");
}

}  // namespace

int hb_gemm_num_configs() { return kNumConfigs; }
bool hb_gemm_config_supports(int id, const hb_gemm_args& a) {
  (void)a;
  return id >= 0 && id < kNumConfigs;
}

void hb_gemm_config_describe(int id, hb_tune_result* out) {
  const GemmVariant& v = kVariants[id / kNumRasters];
  out->config_id = id;
  out->tile_m = v.cluster == 2 ? 256 : BM;
  out->tile_n = v.bn;
  out->tile_k = BK * v.kps;
  out->stages = v.stages;
  out->cluster = v.cluster;
  out->raster_group = kRasters[id % kNumRasters];
  out->split_k = 1;
}

// The configuration with these properties, or -1 (the persisted cache names configurations by
// their properties, so that it survives changes of this table).
int hb_gemm_find_config(int cluster, int tile_n, int tile_k, int stages, int raster_group) {
  for (int id = 0; id < kNumConfigs; ++id) {
    const GemmVariant& v = kVariants[id / kNumRasters];
    if (v.cluster == cluster && v.bn == tile_n && BK * v.kps == tile_k && v.stages == stages &&
        kRasters[id % kNumRasters] == raster_group)
      return id;
  }
  return -1;
}

hb_status hb_launch_gemm_bf16(hb_ctx* ctx, const hb_gemm_args& a, int config_id) {
  if (config_id < 0 || config_id >= kNumConfigs)
    return hb_fail(ctx, HB_ERR_INVALID, "matmul: config_id %d out of range [0,%d)", config_id,
                   kNumConfigs);
  const GemmVariant cfg = kVariants[config_id / kNumRasters];
  const int bn_cta = cfg.cluster == 2 ? cfg.bn / 2 : cfg.bn;     // B rows one CTA loads per k-block
  // K-major operand: dims (K, rows), box (64, rows per CTA); MN-major: dims (rows, K), boxes of (64, 64)
  CUtensorMap tmA, tmB;
  hb_status st;
  uint64_t dimsA[2] = {(uint64_t)(a.a_mn_major ? a.M : a.K), (uint64_t)(a.a_mn_major ? a.K : a.M)};
  uint64_t dimsB[2] = {(uint64_t)(a.b_mn_major ? a.N : a.K), (uint64_t)(a.b_mn_major ? a.K : a.N)};
  uint64_t strA[1] = {(uint64_t)a.lda * 2}, strB[1] = {(uint64_t)a.ldb * 2};
  uint32_t boxA[2] = {64, a.a_mn_major ? 64u : 128u}, boxB[2] = {64, a.b_mn_major ? 64u : (uint32_t)bn_cta};
  if ((st = hb_make_tensor_map(ctx, &tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.A, dimsA, strA, boxA,
                               CU_TENSOR_MAP_SWIZZLE_128B)) != HB_OK) return st;
  if ((st = hb_make_tensor_map(ctx, &tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.B, dimsB, strB, boxB,
                               CU_TENSOR_MAP_SWIZZLE_128B)) != HB_OK) return st;
  // Output through shared memory and TMA (32 x 32 blocks, 64-byte swizzle) whenever the output's
  // base and pitch allow a tensor map; otherwise the row-per-lane stores.  HB_GEMM_TMA_STORE=0
  // keeps the latter.
  CUtensorMap tmC = tmA;
  bool tma_store = (a.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(a.C) & 15) == 0;
  if (tma_store) {
    if (const char* e = getenv("HB_GEMM_TMA_STORE")) tma_store = atoi(e) != 0;
  }
  if (tma_store) {
    uint64_t dimsC[2] = {(uint64_t)(a.epilogue == HB_EPI_SWIGLU ? a.N / 2 : a.N), (uint64_t)a.M};
    uint64_t strC[1] = {(uint64_t)a.ldc * 2};
    uint32_t boxC[2] = {32, 32};
    if ((st = hb_make_tensor_map(ctx, &tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.C, dimsC, strC, boxC,
                                 CU_TENSOR_MAP_SWIZZLE_64B)) != HB_OK) return st;
  }
  GemmParams p;
  p.tma_store = tma_store ? 1 : 0;
  p.C = static_cast<__nv_bfloat16*>(a.C);
  p.R = static_cast<const __nv_bfloat16*>(a.residual);
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.ldc = a.ldc; p.ldr = a.ldr;
  p.raster_group = kRasters[config_id % kNumRasters];
  p.epilogue = a.epilogue;
  p.a_mn = a.a_mn_major; p.b_mn = a.b_mn_major;
  p.status = ctx->d_status;
  p.ready = a.ready; p.ready_epoch = a.ready_epoch; p.ready_spin = a.ready_spin; p.ready_rows = a.ready_rows;
  p.perm_world = 0; p.perm_rank = 0;
  if (a.ready && a.perm_world > 1) {
    const int tile_rows = cfg.cluster == 2 ? 256 : BM;
    const int64_t tiles_m = (a.M + tile_rows - 1) / tile_rows;
    if (a.M % tile_rows == 0 && tiles_m % a.perm_world == 0) { p.perm_world = a.perm_world; p.perm_rank = a.perm_rank; }
  }
#define HB_CASE1(BN, ST, KP) if (cfg.cluster == 1 && cfg.bn == BN && cfg.stages == ST && cfg.kps == KP) return launch_cfg<BN, ST, KP>(ctx, tmA, tmB, tmC, p)
#define HB_CASE2(BN, ST, KP) if (cfg.cluster == 2 && cfg.bn == BN && cfg.stages == ST && cfg.kps == KP) return launch_pair<BN, ST, KP>(ctx, tmA, tmB, tmC, p)
  HB_CASE1(256, 4, 1); HB_CASE1(256, 3, 1); HB_CASE1(256, 2, 2);
  HB_CASE1(128, 6, 1); HB_CASE1(128, 4, 1); HB_CASE1(128, 3, 2);
  HB_CASE1(64, 8, 1);  HB_CASE1(64, 5, 1);  HB_CASE1(64, 4, 2);
  HB_CASE2(256, 6, 1); HB_CASE2(256, 5, 1); HB_CASE2(256, 4, 1); HB_CASE2(256, 3, 2);
  HB_CASE2(128, 8, 1); HB_CASE2(128, 6, 1); HB_CASE2(128, 4, 2);
#undef HB_CASE1
#undef HB_CASE2
  return hb_fail(ctx, HB_ERR_INVALID, "matmul: configuration %d has no kernel", config_id);
}
