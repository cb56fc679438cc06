// Fused causal attention forward for sm_100a, head_dim 128, bf16 in/out.
//   O = softmax(scale * Q K^T + mask) V per (batch, head); fp32 scores, fp32 running
//   max / sum, P rounded to bf16 for the PV product, output normalised once at the end.
//
// One CTA owns 256 query rows of one (batch, head): two 128-row tiles that ping-pong so
// the tensor core works on one tile while the other is in its softmax.
//   warps 0..3   softmax of tile 0: one thread per query row (= one TMEM lane).  Reads the
//   warps 4..7   softmax of tile 1  S row with tcgen05.ld, keeps max / sum in registers,
//                writes P (bf16) back over S with tcgen05.st, rescales O in TMEM only
//                when the row max grew by more than 2^8 (lazy rescale), and finally
//                normalises and stores O.
//   warp 8       TMA producer: Q once, then K and V tiles through two-deep rings.
//   warp 9       MMA issuer: S = Q K^T (both operands K-major in shared memory) and
//                O += P V (P from tensor memory, V MN-major in shared memory).
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_t
// aliases the first 64 columns of S_t.  tcgen05.mma executes in issue order, so the
// commit that publishes S_t(j) also proves O_t += P_t V (j-1) has finished.
//
// Two instantiations.  In the plain one a CTA computes one work unit (blockIdx.x).  In the
// persistent one the grid is one CTA per SM and every CTA pulls units from a global counter
// (the TMA thread fetches, the other roles read the unit from a two-slot shared-memory
// mailbox); barrier phases then run on across units, Q's buffer is handed back as soon as the
// unit's last score product has run, and the next unit's Q, first K/V tiles and first score
// products execute under the current unit's last softmax, PV and output store.
//
// Algorithmic work (causal): 4 * B * H * S^2 * D / 2 flop; traffic (Q + K + V + O) * 2 B.
#include <math.h>
#include <stdlib.h>

#include <algorithm>

#include "hb_internal.h"
#include "hb_ptx.cuh"

namespace {

using namespace hb;

constexpr int D = 128;           // head_dim
constexpr int BQ = 128;          // query rows per tile (two tiles per CTA)
constexpr int BKV = 128;         // keys per KV tile
constexpr int KV_STAGES = 2;
constexpr int ATTN_THREADS = 320;
constexpr int TILE_BYTES = BQ * D * 2;        // 32 KB: two 128-byte-swizzled boxes of 64 columns
constexpr int HALF_BYTES = TILE_BYTES / 2;    // one box: 128 rows x 128 B
constexpr float RESCALE_THRESHOLD = 8.0f;     // in log2 units

struct AttnParams {
  __nv_bfloat16* O;
  float* lse;
  int B, S, Hq, Hkv;
  int64_t o_sb, o_ss, o_sh;     // O strides (elements) for batch, seq, head
  int causal;
  float scale_log2;             // scale * log2(e)
  float scale;
  int n_qblocks;                // ceil(S / 256)
  int n_units;                  // B * Hq * n_qblocks
  int32_t* work_counter;        // persistent kernel: next unit to hand out (zero at launch)
  int32_t* status;
};

struct Smem {
  static constexpr int OFF_Q = 0;                                   // 2 tiles
  static constexpr int OFF_K = OFF_Q + 2 * TILE_BYTES;              // KV_STAGES tiles
  static constexpr int OFF_V = OFF_K + KV_STAGES * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_V + KV_STAGES * TILE_BYTES;
  // q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_ready[2][2 halves], o_full[2],
  // q_empty, unit_full[2], unit_empty[2]
  static constexpr int NUM_BARS = 1 + 4 * KV_STAGES + 8 + 5;
  static constexpr int OFF_UNIT = OFF_BAR + NUM_BARS * 8;           // int unit[2]: the mailbox
  static constexpr int OFF_TMEM_PTR = OFF_UNIT + 8;
  static constexpr int OFF_ABORT = OFF_TMEM_PTR + 4;
  static constexpr int TOTAL = OFF_ABORT + 4;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

template <bool PERSIST>
__global__ void __launch_bounds__(ATTN_THREADS, 1)
hb_attention_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + Smem::OFF_Q;
  const uint32_t sK = smem_base + Smem::OFF_K;
  const uint32_t sV = smem_base + Smem::OFF_V;
  const uint32_t bar0 = smem_base + Smem::OFF_BAR;
  const uint32_t bar_q_full = bar0;
  const uint32_t bar_k_full = bar0 + 8;
  const uint32_t bar_k_empty = bar_k_full + KV_STAGES * 8;
  const uint32_t bar_v_full = bar_k_empty + KV_STAGES * 8;
  const uint32_t bar_v_empty = bar_v_full + KV_STAGES * 8;
  const uint32_t bar_s_full = bar_v_empty + KV_STAGES * 8;
  const uint32_t bar_p_ready = bar_s_full + 2 * 8;
  const uint32_t bar_o_full = bar_p_ready + 4 * 8;
  const uint32_t bar_q_empty = bar_o_full + 2 * 8;
  const uint32_t bar_unit_full = bar_q_empty + 8;
  const uint32_t bar_unit_empty = bar_unit_full + 2 * 8;
  volatile int* unit_box = reinterpret_cast<volatile int*>(smem + Smem::OFF_UNIT);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + Smem::OFF_TMEM_PTR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::OFF_ABORT);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Work unit: heavy (late) query blocks of a head first; the blocks of one head run
  // together so its K/V stay in L2.
  struct Unit { int b, h, hk, q0, n_t[2], n_max; bool tile1_live; };
  auto decode = [&](int unit) {
    Unit u;
    const int bh = unit / p.n_qblocks;
    const int qblk = p.n_qblocks - 1 - (unit % p.n_qblocks);
    u.b = bh / p.Hq;
    u.h = bh % p.Hq;
    u.hk = u.h / (p.Hq / p.Hkv);
    u.q0 = qblk * 2 * BQ;              // first query row of tile 0
    // Number of KV tiles each query tile visits.
    const int n_all = (p.S + BKV - 1) / BKV;
    if (p.causal) {
      u.n_t[0] = min(n_all, (u.q0 + BQ + BKV - 1) / BKV);
      u.n_t[1] = min(n_all, (u.q0 + 2 * BQ + BKV - 1) / BKV);
    } else {
      u.n_t[0] = u.n_t[1] = n_all;
    }
    u.tile1_live = (u.q0 + BQ) < p.S;  // tile 1 may lie wholly past the sequence
    if (!u.tile1_live) u.n_t[1] = 0;
    u.n_max = max(u.n_t[0], u.n_t[1]);
    return u;
  };
  // Consumers of the mailbox: unit number `uq` of this CTA.  The MMA thread calls it alone
  // (`whole_warp` false); a softmax warp calls it with all lanes, every lane waits and reads,
  // and lane 0 (`arrive`) hands the slot back once all of them have.
  auto next_unit = [&](int uq, bool whole_warp, bool arrive, bool& ok) -> int {
    if (!PERSIST) return uq == 0 ? (int)blockIdx.x : p.n_units;
    const int slot = uq & 1;
    if (!mbar_wait(bar_unit_full + slot * 8, (uq >> 1) & 1, abort_flag)) { ok = false; return p.n_units; }
    const int unit = unit_box[slot];
    if (whole_warp) __syncwarp();
    if (arrive) mbar_arrive(bar_unit_empty + slot * 8);
    return unit;
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(bar_k_full + s * 8, 1);
      mbar_init(bar_k_empty + s * 8, 1);
      mbar_init(bar_v_full + s * 8, 1);
      mbar_init(bar_v_empty + s * 8, 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_s_full + t * 8, 1);
      mbar_init(bar_p_ready + (t * 2) * 8, 4);        // one arrival per softmax warp of the tile
      mbar_init(bar_p_ready + (t * 2 + 1) * 8, 4);
      mbar_init(bar_o_full + t * 8, 1);
    }
    mbar_init(bar_q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_unit_full + i * 8, 1);
      mbar_init(bar_unit_empty + i * 8, 9);           // MMA thread + one lane of each softmax warp
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 9) {
    tmem_alloc<1>(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), 512);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer (+ unit hand-out)
    if (elect_one()) {
      bool ok = true;
      int g = 0;                                  // KV tiles loaded so far by this CTA: ring position
      for (int uq = 0; ok; ++uq) {
        int unit;
        if (PERSIST) {
          const int slot = uq & 1;
          if (!mbar_wait(bar_unit_empty + slot * 8, ((uq >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
          unit = atomicAdd(p.work_counter, 1);
          if (unit > p.n_units) unit = p.n_units;
          unit_box[slot] = unit;
          mbar_arrive(bar_unit_full + slot * 8);
        } else {
          unit = uq == 0 ? (int)blockIdx.x : p.n_units;
        }
        if (unit >= p.n_units) break;
        const Unit u = decode(unit);
        // Q's buffer is free once the previous unit's last score product has run.
        if (!mbar_wait(bar_q_empty, (uq & 1) ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(bar_q_full, (u.tile1_live ? 2 : 1) * TILE_BYTES);
        for (int t = 0; t < (u.tile1_live ? 2 : 1); ++t)
          for (int c = 0; c < 2; ++c)
            tma_load_4d(sQ + t * TILE_BYTES + c * HALF_BYTES, &tmQ, bar_q_full, c * 64, u.h, u.q0 + t * BQ, u.b);
        for (int j = 0; j < u.n_max && ok; ++j, ++g) {
          const int s = g % KV_STAGES;
          const uint32_t ph = (g / KV_STAGES) & 1;
          if (!mbar_wait(bar_k_empty + s * 8, ph ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(bar_k_full + s * 8, TILE_BYTES);
          for (int c = 0; c < 2; ++c)
            tma_load_4d(sK + s * TILE_BYTES + c * HALF_BYTES, &tmK, bar_k_full + s * 8, c * 64, u.hk, j * BKV, u.b);
          if (!mbar_wait(bar_v_empty + s * 8, ph ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(bar_v_full + s * 8, TILE_BYTES);
          for (int c = 0; c < 2; ++c)
            tma_load_4d(sV + s * TILE_BYTES + c * HALF_BYTES, &tmV, bar_v_full + s * 8, c * 64, u.hk, j * BKV, u.b);
        }
      }
      if (!ok && p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_ATTN; p.status[2] = 1; }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_qk = umma_idesc_bf16(BQ, BKV, 0, 0);
      const uint32_t idesc_pv = umma_idesc_bf16(BQ, D, 0, 1);
      bool ok = true;
      // Descriptors are built once; inside the loops only the 14-bit start-address field
      // (bytes >> 4, in the low word) moves, by constants that cannot carry out of it.
      const uint64_t desc_q = umma_desc_k_sw128(sQ);
      const uint64_t desc_k = umma_desc_k_sw128(sK);
      const uint64_t desc_v = umma_desc_mn_sw128(sV, HALF_BYTES, 1024);
      auto issue_qk = [&](int t, int g) {          // g: ring position of the K tile
        const int s = g % KV_STAGES;
        const uint32_t d_tmem = tmem_base + t * 128;
        const uint64_t a_desc = desc_q + static_cast<uint32_t>(t * (TILE_BYTES >> 4));
        const uint64_t b_desc = desc_k + static_cast<uint32_t>(s * (TILE_BYTES >> 4));
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * HALF_BYTES + (kk & 3) * 32) >> 4;
          umma_ss<1>(d_tmem, a_desc + off, b_desc + off, idesc_qk, kk != 0 ? 1u : 0u);
        }
        umma_commit<1>(bar_s_full + t * 8);
      };
      auto issue_pv = [&](int t, int g, int j, int hf) {     // keys [64 hf, 64 hf + 64) of KV tile j of the unit
        const int s = g % KV_STAGES;
        const uint32_t d_tmem = tmem_base + 256 + t * 128;
        const uint32_t a_tmem = tmem_base + t * 128;     // P aliases S: 64 packed columns
        const uint64_t b_desc = desc_v + static_cast<uint32_t>(s * (TILE_BYTES >> 4));
#pragma unroll
        for (int kk = hf * 4; kk < hf * 4 + 4; ++kk)
          umma_ts(d_tmem, a_tmem + kk * 8, b_desc + static_cast<uint32_t>(kk * (2048 >> 4)), idesc_pv,
                  (j | kk) != 0 ? 1u : 0u);
      };
      int g0 = 0;                                  // ring position of the unit's first KV tile
      uint32_t np[2] = {0, 0};                     // P publications consumed per tile: barrier phase
      for (int uq = 0; ok; ++uq) {
        const int unit = next_unit(uq, false, true, ok);
        if (!ok || unit >= p.n_units) break;
        const Unit u = decode(unit);
        if (!mbar_wait(bar_q_full, uq & 1, abort_flag)) { ok = false; break; }
        // Prologue: S_t(0) for both tiles.
        if (!mbar_wait(bar_k_full + (g0 % KV_STAGES) * 8, (g0 / KV_STAGES) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        issue_qk(0, g0);
        if (u.n_t[1] > 0) issue_qk(1, g0);
        umma_commit<1>(bar_k_empty + (g0 % KV_STAGES) * 8);   // K(0) is free once both S(0) products have read it
        if (u.n_max <= 1) umma_commit<1>(bar_q_empty);
        for (int j = 0; j < u.n_max && ok; ++j) {
          const int g = g0 + j;
          const int s = g % KV_STAGES;
          const uint32_t ph = (g / KV_STAGES) & 1;
          const int sn = (g + 1) % KV_STAGES;
          const uint32_t phn = ((g + 1) / KV_STAGES) & 1;
          if (!mbar_wait(bar_v_full + s * 8, ph, abort_flag)) { ok = false; break; }
          if (j + 1 < u.n_max && !mbar_wait(bar_k_full + sn * 8, phn, abort_flag)) { ok = false; break; }
          for (int t = 0; t < 2; ++t) {
            if (j < u.n_t[t]) {
              if (!mbar_wait_spin(bar_p_ready + (t * 2) * 8, np[t] & 1, abort_flag)) { ok = false; break; }
              tc_fence_after();
              issue_pv(t, g, j, 0);
              if (!mbar_wait_spin(bar_p_ready + (t * 2 + 1) * 8, np[t] & 1, abort_flag)) { ok = false; break; }
              tc_fence_after();
              issue_pv(t, g, j, 1);
              ++np[t];
              if (j + 1 == u.n_t[t]) umma_commit<1>(bar_o_full + t * 8);
            }
            if (j + 1 < u.n_t[t]) issue_qk(t, g + 1);
          }
          if (!ok) break;
          umma_commit<1>(bar_v_empty + s * 8);
          if (j + 1 < u.n_max) umma_commit<1>(bar_k_empty + sn * 8);
          if (j + 2 == u.n_max) umma_commit<1>(bar_q_empty);   // every score product of the unit has been issued
        }
        g0 += u.n_max;
      }
      if (!ok && p.status) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_ATTN; p.status[2] = 2; }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int t = warp >> 2;                    // query tile of this warpgroup
    const int qd = warp & 3;                    // TMEM lane quarter
    const int r = qd * 32 + lane;               // row within the tile
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const uint32_t tS = tmem_base + lane_off + t * 128;
    const uint32_t tO = tmem_base + lane_off + 256 + t * 128;
    bool ok = true;
    uint32_t ns = 0;                            // S tiles consumed by this warp: barrier phase
    uint32_t no = 0;                            // units whose O this warp has stored
    for (int uq = 0; ok; ++uq) {
    const int unit = next_unit(uq, true, lane == 0, ok);
    if (!ok || unit >= p.n_units) break;
    const Unit u = decode(unit);
    const int row = u.q0 + t * BQ + r;          // global query row
    const int b = u.b, h = u.h;
    float m_ref = -INFINITY;                    // reference max (raw score units)
    float l = 0.f;                              // running sum of exp2
    const int n_mine = u.n_t[t];
    for (int j = 0; j < n_mine && ok; ++j, ++ns) {
      if (!mbar_wait(bar_s_full + t * 8, ns & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t(&chunk)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[c * 32]);
        tmem_ld_32x32(tS + c * 32, chunk);
      }
      tmem_wait_ld();
      // Mask: keys past the sequence end, and (diagonal tile) keys after this query.
      const int k0 = j * BKV;
      int limit = p.S - 1 - k0;
      if (p.causal) limit = min(limit, row - k0);
      if (limit < BKV - 1) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i > limit) sv[i] = 0xff800000u;   // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(sv[i]));
        mx1 = fmaxf(mx1, __uint_as_float(sv[i + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(sv[i + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(sv[i + 3]));
      }
      const float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      // Lazy rescale: move the reference max only when it would grow by more than 2^8.
      bool need = (m_tile - m_ref) * p.scale_log2 > RESCALE_THRESHOLD;   // true on the first tile
      if (m_tile == -INFINITY) need = false;
      float factor = 1.0f;
      if (need) {
        factor = (m_ref == -INFINITY) ? 0.0f : ex2_approx((m_ref - m_tile) * p.scale_log2);
        m_ref = m_tile;
        l *= factor;
      }
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        // O_t += P V (j-1) has completed (see header); rescale this warp's 32 rows.
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(tO + c * 32, ov);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * factor);
          tmem_st_32x32(tO + c * 32, ov);
        }
      }
      const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref * p.scale_log2;
      // P is produced and published in two halves of 64 keys: the PV product starts on the
      // first half while the second is still being exponentiated.
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int e = hf * 64 + 2 * i;
          const float e0 = ex2_approx(fmaf(__uint_as_float(sv[e]), p.scale_log2, neg_m));
          const float e1 = ex2_approx(fmaf(__uint_as_float(sv[e + 1]), p.scale_log2, neg_m));
          const float e2 = ex2_approx(fmaf(__uint_as_float(sv[e + 2]), p.scale_log2, neg_m));
          const float e3 = ex2_approx(fmaf(__uint_as_float(sv[e + 3]), p.scale_log2, neg_m));
          l0 += e0; l1 += e1; l2 += e2; l3 += e3;
          pk[i] = pack_bf16x2(e0, e1);
          pk[i + 1] = pack_bf16x2(e2, e3);
        }
        tmem_st_32x32(tS + hf * 32, pk);     // 32 packed columns = 64 keys
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_ready + (t * 2 + hf) * 8);
      }
      l += (l0 + l1) + (l2 + l3);
    }
    // ---- epilogue: O / l -> bf16 -> global
    if (ok && n_mine > 0) {
      if (!mbar_wait(bar_o_full + t * 8, no & 1, abort_flag)) ok = false;
      ++no;
    }
    if (ok && n_mine > 0) {
      tc_fence_after();
      const float inv_l = 1.0f / l;
      __nv_bfloat16* dst = p.O + b * p.o_sb + static_cast<int64_t>(row) * p.o_ss + h * p.o_sh;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t ov[32];
        tmem_ld_32x32(tO + c * 32, ov);
        tmem_wait_ld();
        if (row < p.S) {
          uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(ov[8 * i + 0]) * inv_l, __uint_as_float(ov[8 * i + 1]) * inv_l);
            o.y = pack_bf16x2(__uint_as_float(ov[8 * i + 2]) * inv_l, __uint_as_float(ov[8 * i + 3]) * inv_l);
            o.z = pack_bf16x2(__uint_as_float(ov[8 * i + 4]) * inv_l, __uint_as_float(ov[8 * i + 5]) * inv_l);
            o.w = pack_bf16x2(__uint_as_float(ov[8 * i + 6]) * inv_l, __uint_as_float(ov[8 * i + 7]) * inv_l);
            d4[i] = o;
          }
        }
      }
      if (p.lse && row < p.S)
        p.lse[(static_cast<int64_t>(b) * p.Hq + h) * p.S + row] = m_ref * p.scale + logf(l);
    }
    }   // units
    if (!ok && p.status && lane == 0) { atomicCAS(p.status, 0, HB_ERR_TIMEOUT); p.status[1] = HB_KTAG_ATTN; p.status[2] = 3; }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

hb_status make_qkv_map(hb_ctx* ctx, CUtensorMap* m, const hb_tensor* t) {
  // dims innermost first: (D, H, S, B); box (64, 1, 128, 1)
  uint64_t dims[4] = {(uint64_t)t->shape[3], (uint64_t)t->shape[2], (uint64_t)t->shape[1], (uint64_t)t->shape[0]};
  uint64_t strides[3] = {(uint64_t)t->stride[2] * 2, (uint64_t)t->stride[1] * 2, (uint64_t)t->stride[0] * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return hb_make_tensor_map(ctx, m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t->ptr, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

extern "C" hb_status hb_attention(hb_ctx* ctx, const hb_tensor* Q, const hb_tensor* K, const hb_tensor* V,
                                  hb_tensor* O, const hb_attn_opts* opts) {
  if (!ctx) return HB_ERR_INVALID;
  if (!Q || !K || !V || !O || !opts) return hb_fail(ctx, HB_ERR_INVALID, "attention: null argument");
  const hb_tensor* ts[4] = {Q, K, V, O};
  for (const hb_tensor* t : ts) {
    if (t->rank != 4) return hb_fail(ctx, HB_ERR_INVALID, "attention: tensors must be [batch, seq, heads, head_dim]");
    if (t->dtype != HB_BF16) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "attention: only bf16 is supported");
    if (!t->ptr) return hb_fail(ctx, HB_ERR_INVALID, "attention: null data pointer");
    if (t->stride[3] != 1) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "attention: head_dim must be contiguous");
    if ((t->stride[0] | t->stride[1] | t->stride[2]) & 7)
      return hb_fail(ctx, HB_ERR_UNSUPPORTED, "attention: strides must be multiples of 8 elements");
    if (reinterpret_cast<uintptr_t>(t->ptr) & 15)
      return hb_fail(ctx, HB_ERR_INVALID, "attention: data pointers must be 16-byte aligned");
  }
  const int64_t B = Q->shape[0], S = Q->shape[1], Hq = Q->shape[2], Dh = Q->shape[3];
  const int64_t Hkv = K->shape[2];
  if (Dh != D) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "attention: head_dim must be 128 (got %lld)", (long long)Dh);
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0) return hb_fail(ctx, HB_ERR_INVALID, "attention: empty dimension");
  if (Hq % Hkv) return hb_fail(ctx, HB_ERR_INVALID, "attention: %lld query heads not a multiple of %lld KV heads",
                               (long long)Hq, (long long)Hkv);
  if (K->shape[0] != B || K->shape[1] != S || K->shape[3] != D || V->shape[0] != B || V->shape[1] != S ||
      V->shape[2] != Hkv || V->shape[3] != D)
    return hb_fail(ctx, HB_ERR_INVALID, "attention: K and V must be [batch, seq, kv_heads, 128]");
  for (int i = 0; i < 4; ++i)
    if (O->shape[i] != Q->shape[i]) return hb_fail(ctx, HB_ERR_INVALID, "attention: O must be shaped like Q");
  if (!(opts->scale > 0.f) || !isfinite(opts->scale))
    return hb_fail(ctx, HB_ERR_INVALID, "attention: scale must be positive and finite");
  if (S > (1 << 24)) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "attention: sequence too long");

  CUtensorMap tmQ, tmK, tmV;
  hb_status st;
  if ((st = make_qkv_map(ctx, &tmQ, Q)) != HB_OK) return st;
  if ((st = make_qkv_map(ctx, &tmK, K)) != HB_OK) return st;
  if ((st = make_qkv_map(ctx, &tmV, V)) != HB_OK) return st;

  AttnParams p;
  p.O = static_cast<__nv_bfloat16*>(O->ptr);
  p.lse = static_cast<float*>(opts->lse);
  p.B = (int)B; p.S = (int)S; p.Hq = (int)Hq; p.Hkv = (int)Hkv;
  p.o_sb = O->stride[0]; p.o_ss = O->stride[1]; p.o_sh = O->stride[2];
  p.causal = opts->causal ? 1 : 0;
  p.scale = opts->scale;
  p.scale_log2 = opts->scale * 1.4426950408889634f;
  p.n_qblocks = (int)((S + 2 * BQ - 1) / (2 * BQ));
  p.status = ctx->d_status;
  const int64_t units = B * Hq * p.n_qblocks;
  if (units >= INT32_MAX - 4096) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "attention: too many work units");
  p.n_units = (int)units;
  // Persistent form when every SM would otherwise run several CTAs in a row; the environment
  // variable HB_ATTN_PERSISTENT=0/1 overrides.  Each launch takes the next of a few work
  // counters so that launches in flight on different streams never share one.
  bool persist = units >= 2 * (int64_t)ctx->sm_count;
  if (opts->config_id == 0 || opts->config_id == 1) {
    persist = opts->config_id == 1;                       // the caller's choice (the autotuner's candidates)
  } else {
    const int cached = hb_attention_cached_choice(ctx, B, S, Hq, Hkv, opts->causal ? 1 : 0);
    if (cached == 0 || cached == 1) persist = cached == 1;
  }
  if (const char* e = getenv("HB_ATTN_PERSISTENT")) persist = atoi(e) != 0;
  p.work_counter = nullptr;
  if (persist) {
    p.work_counter = ctx->d_status + 8 + (ctx->attn_launches++ & 7);
    cudaError_t e = cudaMemsetAsync(p.work_counter, 0, sizeof(int32_t), ctx->stream);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaMemsetAsync(attention work counter)");
  }
  const int64_t grid = persist ? std::min<int64_t>(units, ctx->sm_count) : units;

  static bool attr_set[64] = {};
  if (!attr_set[ctx->device & 63]) {
    cudaError_t e = cudaFuncSetAttribute(hb_attention_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Smem::DYN_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(hb_attention_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               Smem::DYN_BYTES);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaFuncSetAttribute(attention)");
    attr_set[ctx->device & 63] = true;
  }
  if (persist)
    hb_attention_fwd_kernel<true><<<(unsigned)grid, ATTN_THREADS, Smem::DYN_BYTES, ctx->stream>>>(tmQ, tmK, tmV, p);
  else
    hb_attention_fwd_kernel<false><<<(unsigned)grid, ATTN_THREADS, Smem::DYN_BYTES, ctx->stream>>>(tmQ, tmK, tmV, p);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "attention launch");
}

extern "C" hb_status hb_attention_host(hb_ctx* ctx, const void* Q, const void* K, const void* V, void* O,
                                       int64_t batch, int64_t seq, int64_t n_q_heads, int64_t n_kv_heads,
                                       int64_t head_dim, int32_t causal, float scale) {
  if (!ctx) return HB_ERR_INVALID;
  if (!Q || !K || !V || !O) return hb_fail(ctx, HB_ERR_INVALID, "attention_host: null buffer");
  if (batch <= 0 || seq <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0)
    return hb_fail(ctx, HB_ERR_INVALID, "attention_host: empty dimension");
  const size_t q_b = (size_t)batch * seq * n_q_heads * head_dim * 2;
  const size_t kv_b = (size_t)batch * seq * n_kv_heads * head_dim * 2;
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  void* base = nullptr;
  hb_status st = hb_get_scratch(ctx, HB_SCRATCH_STAGING, 2 * up(q_b) + 2 * up(kv_b), &base);
  if (st != HB_OK) return st;
  char* dQ = static_cast<char*>(base);
  char* dK = dQ + up(q_b);
  char* dV = dK + up(kv_b);
  char* dO = dV + up(kv_b);
  const int64_t q_row = seq * n_q_heads * head_dim, kv_row = seq * n_kv_heads * head_dim;   // elements per batch entry
  auto mk = [&](char* ptr, int64_t heads, int64_t b0, int64_t nb) {
    hb_tensor t = {ptr + (size_t)b0 * seq * heads * head_dim * 2, HB_BF16, 4, {nb, seq, heads, head_dim},
                   {seq * heads * head_dim, heads * head_dim, head_dim, 1}};
    return t;
  };
  hb_attn_opts opts = {causal, scale, nullptr, -1};
  // Batch entries are independent, so large calls are pipelined over groups of them: copy-in
  // of group i+1 and copy-out of group i-1 run under the kernel of group i.
  const int chunks = (batch >= 2 && q_b >= (size_t(8) << 20)) ? (int)(batch < 8 ? batch : 8) : 1;
  if (chunks == 1) {
    if ((st = hb_upload(ctx, dQ, Q, q_b)) != HB_OK) return st;
    if ((st = hb_upload(ctx, dK, K, kv_b)) != HB_OK) return st;
    if ((st = hb_upload(ctx, dV, V, kv_b)) != HB_OK) return st;
    hb_tensor tQ = mk(dQ, n_q_heads, 0, batch), tK = mk(dK, n_kv_heads, 0, batch);
    hb_tensor tV = mk(dV, n_kv_heads, 0, batch), tO = mk(dO, n_q_heads, 0, batch);
    if ((st = hb_attention(ctx, &tQ, &tK, &tV, &tO, &opts)) != HB_OK) return st;
    if ((st = hb_download(ctx, O, dO, q_b)) != HB_OK) return st;
    return hb_sync(ctx);
  }
  cudaEvent_t* ev = nullptr;
  if ((st = hb_host_pipe(ctx, 2 * chunks + 2, &ev)) != HB_OK) return st;
  cudaEvent_t ev_start = ev[2 * chunks], ev_done = ev[2 * chunks + 1];
  const int64_t per = (batch + chunks - 1) / chunks;
  HB_CUDA(ctx, cudaEventRecord(ev_start, ctx->stream));
  HB_CUDA(ctx, cudaStreamWaitEvent(ctx->h2d_stream, ev_start, 0));
  HB_CUDA(ctx, cudaStreamWaitEvent(ctx->d2h_stream, ev_start, 0));
  for (int i = 0; i < chunks; ++i) {
    const int64_t b0 = i * per, nb = (b0 + per <= batch ? per : batch - b0);
    if (nb <= 0) { HB_CUDA(ctx, cudaEventRecord(ev[i], ctx->h2d_stream)); continue; }
    const size_t qo = (size_t)b0 * q_row * 2, ko = (size_t)b0 * kv_row * 2;
    HB_CUDA(ctx, cudaMemcpyAsync(dQ + qo, static_cast<const char*>(Q) + qo, (size_t)nb * q_row * 2,
                                 cudaMemcpyHostToDevice, ctx->h2d_stream));
    HB_CUDA(ctx, cudaMemcpyAsync(dK + ko, static_cast<const char*>(K) + ko, (size_t)nb * kv_row * 2,
                                 cudaMemcpyHostToDevice, ctx->h2d_stream));
    HB_CUDA(ctx, cudaMemcpyAsync(dV + ko, static_cast<const char*>(V) + ko, (size_t)nb * kv_row * 2,
                                 cudaMemcpyHostToDevice, ctx->h2d_stream));
    HB_CUDA(ctx, cudaEventRecord(ev[i], ctx->h2d_stream));
  }
  for (int i = 0; i < chunks; ++i) {
    const int64_t b0 = i * per, nb = (b0 + per <= batch ? per : batch - b0);
    if (nb <= 0) continue;
    HB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ev[i], 0));
    hb_tensor tQ = mk(dQ, n_q_heads, b0, nb), tK = mk(dK, n_kv_heads, b0, nb);
    hb_tensor tV = mk(dV, n_kv_heads, b0, nb), tO = mk(dO, n_q_heads, b0, nb);
    if ((st = hb_attention(ctx, &tQ, &tK, &tV, &tO, &opts)) != HB_OK) return st;
    HB_CUDA(ctx, cudaEventRecord(ev[chunks + i], ctx->stream));
    HB_CUDA(ctx, cudaStreamWaitEvent(ctx->d2h_stream, ev[chunks + i], 0));
    const size_t qo = (size_t)b0 * q_row * 2;
    HB_CUDA(ctx, cudaMemcpyAsync(static_cast<char*>(O) + qo, dO + qo, (size_t)nb * q_row * 2,
                                 cudaMemcpyDeviceToHost, ctx->d2h_stream));
  }
  HB_CUDA(ctx, cudaEventRecord(ev_done, ctx->d2h_stream));
  HB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ev_done, 0));
  return hb_sync(ctx);
}
