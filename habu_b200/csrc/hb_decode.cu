// Decode-shaped path: one new token per sequence against a key/value cache.
//
//   hb_rope_append        rotates the new token's query and key heads at the current position
//                         (same angles as the prefill table: formed and reduced in double) and
//                         appends the rotated keys and the values to the cache;
//   hb_attention_decode   single-query attention over the cache, split along the cached
//                         positions so that a handful of sequences still fills the GPU; the
//                         CTA that finishes a (sequence, KV head) last merges the splits in
//                         split order, so the result does not depend on scheduling;
//   hb_advance_pos        position += n on the device (the step graph is the same every token).
//
// Cache layout: kv[2 * batch, s_max, kv_heads, 128] bf16, keys in the first `batch` entries,
// values in the second -- token-major like every other activation here, so a cache filled by
// the prefill attention's K and V views needs no re-layout.  The position lives in device
// memory (one int32 shared by all sequences): nothing about a step changes on the host, which
// is what lets a planned step be captured once and replayed.
//
// HBM-bound: per step the kernel reads 2 * batch * len * kv_heads * 256 B of cache once.
#include <math.h>

#include "hb_internal.h"

namespace {

constexpr int DD = 128;            // head_dim
constexpr int DEC_TILE = 64;       // cached positions per shared-memory tile (16 per warp)
constexpr int DEC_STAGES = 3;      // tiles in flight per CTA
constexpr int DEC_THREADS = 128;
constexpr int DEC_MAX_G = 8;       // query heads per KV head
constexpr int KV_ROW = DD + 8;     // bf16 per K / V row in shared memory: 272 B, so that the eight
                                   // 16-byte rows of an ldmatrix fall into eight different bank groups
constexpr float DEC_RESCALE = 8.0f;   // the running reference moves only when the maximum grew by 2^8

struct DecodeParams {
  const __nv_bfloat16* qkv;        // [batch, row_stride]: q heads, then k heads, then v heads of the new token
  const __nv_bfloat16* kv;         // cache
  __nv_bfloat16* out;              // [batch, hq * 128]
  float* part_o;                   // [batch * hkv * splits * G][128]
  float* part_ml;                  // [batch * hkv * splits * G][2]  (reference max in log2 units, sum)
  int* tickets;                    // [batch * hkv], zero between launches
  const int32_t* pos;              // current position: the cache holds pos + 1 tokens
  int64_t row_stride;
  int batch, hq, hkv, G, s_max, splits, chunk;   // chunk: positions per split (multiple of DEC_TILE)
  float scale_log2;
  int32_t* status;
};

__device__ __forceinline__ void cp_async16(uint32_t smem, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D(16x8, fp32) += A(16x16, bf16, row) . B(16x8, bf16, col).  Rows 8..15 of A are padding here
// (a1 = a3 = 0): the query heads of one KV head, at most eight, are the rows 0..7.
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct DecSmem {
  __nv_bfloat16 k[DEC_STAGES][DEC_TILE][KV_ROW];
  __nv_bfloat16 v[DEC_STAGES][DEC_TILE][KV_ROW];
  float wml[DEC_THREADS / 32][DEC_MAX_G][2];      // per-warp (reference max, sum)
  int last;
};
// The per-warp partial outputs, merged at the end, reuse the K tiles' memory (the loop is over).
typedef float DecWarpOut[DEC_MAX_G][DD];
static_assert(sizeof(DecWarpOut) * (DEC_THREADS / 32) <= sizeof(__nv_bfloat16) * DEC_STAGES * DEC_TILE * KV_ROW, "merge buffer");

// The cache is read once from HBM; the arithmetic (two small products per cached position) would
// keep the CUDA cores busy three times as long as the read takes, so it runs on the tensor
// cores: per warp and 16 cached positions S[q, pos] = Q K^T and O[q, :] += P V as m16n8k16 tiles
// whose 16 rows hold the (at most eight) query heads that share the KV head -- one pass over K
// and V serves the whole group.  Fragments come from shared memory with ldmatrix (transposed
// for V); P goes from the S accumulators straight into the A operand of the second product.
// The four warps of a CTA take a quarter of every 64-position tile each and keep their own
// running maximum, sum and output, merged at the end in warp order; the CTAs that share a
// (sequence, KV head) are merged in split order by the last one to finish.
__global__ void __launch_bounds__(DEC_THREADS)
hb_attention_decode_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) uint8_t dec_smem_raw[];
  DecSmem& sm = *reinterpret_cast<DecSmem*>(dec_smem_raw);
  // programmatic dependent launch: wait for the kernel in front (RoPE + append) before the first
  // memory access; the attention-out product behind this kernel may start streaming its weights in
  asm volatile("griddepcontrol.wait;\n\tgriddepcontrol.launch_dependents;" ::: "memory");
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int g = lane >> 2, tq = lane & 3;        // fragment row (query head) and column pair
  const int G = p.G;
  int len = *p.pos + 1;
  if (len > p.s_max) len = p.s_max;        // the append kernel has already reported the overflow
  const int begin = split * p.chunk;
  const int end = min(begin + p.chunk, len);
  const int64_t slot = (static_cast<int64_t>(b) * p.hkv + hk) * p.splits + split;

  float o[DD / 8][4];
#pragma unroll
  for (int n = 0; n < DD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m_ref = -INFINITY, l = 0.f;

  if (begin < end) {
    // A fragments of Q for the eight 16-wide chunks of the head dimension: row g = query head g
    uint32_t qa[DD / 16][2];
    {
      const __nv_bfloat16* qrow = p.qkv + b * p.row_stride + static_cast<int64_t>(hk * G + g) * DD;
#pragma unroll
      for (int c = 0; c < DD / 16; ++c) {
        qa[c][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + 16 * c + 2 * tq) : 0u;
        qa[c][1] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + 16 * c + 8 + 2 * tq) : 0u;
      }
    }
    const __nv_bfloat16* kbase = p.kv + (static_cast<int64_t>(b) * p.s_max * p.hkv + hk) * DD;
    const __nv_bfloat16* vbase = p.kv + (static_cast<int64_t>(p.batch + b) * p.s_max * p.hkv + hk) * DD;
    const int64_t pos_stride = static_cast<int64_t>(p.hkv) * DD;
    const int n_tiles = (end - begin + DEC_TILE - 1) / DEC_TILE;
    auto load_tile = [&](int tile) {
      if (tile < n_tiles) {
        const int buf = tile % DEC_STAGES;
        const int p0 = begin + tile * DEC_TILE;
        // 64 rows x 16 chunks of 16 B for K and for V; rows past the end repeat the last valid row
        // (they are masked below; the cache beyond `len` may hold anything, NaN patterns included)
#pragma unroll
        for (int i = 0; i < (DEC_TILE * 16) / DEC_THREADS; ++i) {
          const int idx = t + i * DEC_THREADS;
          const int r = idx >> 4, c = idx & 15;
          const int pos = min(p0 + r, end - 1);
          cp_async16(static_cast<uint32_t>(__cvta_generic_to_shared(&sm.k[buf][r][c * 8])), kbase + pos * pos_stride + c * 8);
          cp_async16(static_cast<uint32_t>(__cvta_generic_to_shared(&sm.v[buf][r][c * 8])), vbase + pos * pos_stride + c * 8);
        }
      }
      cp_async_commit();                                 // an empty group keeps the count uniform
    };
#pragma unroll
    for (int s = 0; s < DEC_STAGES - 1; ++s) load_tile(s);
    for (int tile = 0; tile < n_tiles; ++tile) {
      cp_async_wait<DEC_STAGES - 2>();
      __syncthreads();                                   // tile landed; everyone is done with the buffer refilled next
      load_tile(tile + DEC_STAGES - 1);
      const int buf = tile % DEC_STAGES;
      const int r0 = warp * 16;                          // this warp's 16 positions of the tile
      // ---- S = Q K^T: two 8-position column blocks
      float sacc[2][4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
#pragma unroll
        for (int i = 0; i < DD / 32; ++i) {
          uint32_t kf[4];
          ldsm_x4(static_cast<uint32_t>(__cvta_generic_to_shared(&sm.k[buf][r0 + 8 * nb + (lane & 7)][32 * i + 8 * (lane >> 3)])), kf);
          mma_16816(sacc[nb], qa[2 * i][0], qa[2 * i][1], kf[0], kf[1]);
          mma_16816(sacc[nb], qa[2 * i + 1][0], qa[2 * i + 1][1], kf[2], kf[3]);
        }
      }
      // ---- online softmax for query head g (lanes with g < G): positions r0 + 8 nb + 2 tq, + 1
      const int pg = begin + tile * DEC_TILE + r0 + 2 * tq;
      float sv[4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e)
          sv[2 * nb + e] = (pg + 8 * nb + e < end) ? sacc[nb][e] * p.scale_log2 : -INFINITY;
      float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const bool need = mx > m_ref + DEC_RESCALE || (m_ref == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, need)) {
        if (need) {
          const float f = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx);
          l *= f;
#pragma unroll
          for (int n = 0; n < DD / 8; ++n) { o[n][0] *= f; o[n][1] *= f; }
          m_ref = mx;
        }
      }
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pv[e] = m_ref == -INFINITY ? 0.f : exp2f(sv[e] - m_ref);     // masked positions: exp2(-inf) = 0
        l += pv[e];
      }
      const uint32_t pa0 = g < G ? pack2_bf16(pv[0], pv[1]) : 0u;     // positions 2 tq, 2 tq + 1
      const uint32_t pa2 = g < G ? pack2_bf16(pv[2], pv[3]) : 0u;     // positions 8 + 2 tq, + 1
      // ---- O += P V: sixteen 8-wide column blocks of the head dimension
#pragma unroll
      for (int n = 0; n < DD / 16; ++n) {
        uint32_t vf[4];
        ldsm_x4_trans(static_cast<uint32_t>(__cvta_generic_to_shared(
                          &sm.v[buf][r0 + 8 * ((lane >> 3) & 1) + (lane & 7)][16 * n + 8 * (lane >> 4)])), vf);
        mma_16816(o[2 * n], pa0, pa2, vf[0], vf[1]);
        mma_16816(o[2 * n + 1], pa0, pa2, vf[2], vf[3]);
      }
    }
    cp_async_wait<0>();
  }
  // ---- merge the four warps (warp order), then publish this split's partial result
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  __syncthreads();                                       // every warp has read its last tile
  DecWarpOut* wo = reinterpret_cast<DecWarpOut*>(&sm.k[0][0][0]);
  if (g < G) {
#pragma unroll
    for (int n = 0; n < DD / 8; ++n) {
      wo[warp][g][8 * n + 2 * tq] = o[n][0];
      wo[warp][g][8 * n + 2 * tq + 1] = o[n][1];
    }
    if (tq == 0) { sm.wml[warp][g][0] = m_ref; sm.wml[warp][g][1] = l; }
  }
  __syncthreads();
  for (int q = 0; q < G; ++q) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) M = fmaxf(M, sm.wml[w][q][0]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) {
      const float lw = sm.wml[w][q][1];
      const float wgt = lw > 0.f ? exp2f(sm.wml[w][q][0] - M) : 0.f;
      L += lw * wgt;
      acc += wo[w][q][t] * wgt;
    }
    p.part_o[(slot * G + q) * DD + t] = acc;
    if (t == 0) {
      p.part_ml[(slot * G + q) * 2] = M;
      p.part_ml[(slot * G + q) * 2 + 1] = L;
    }
  }
  __threadfence();
  __syncthreads();
  if (t == 0) {
    const int arrived = atomicAdd(&p.tickets[b * p.hkv + hk], 1);
    sm.last = arrived == p.splits - 1;
  }
  __syncthreads();
  if (!sm.last) return;
  __threadfence();
  // ---- merge the splits, in split order
  const int64_t first = (static_cast<int64_t>(b) * p.hkv + hk) * p.splits;
  for (int q = 0; q < G; ++q) {
    float M = -INFINITY;
    for (int s = 0; s < p.splits; ++s) M = fmaxf(M, __ldcg(&p.part_ml[((first + s) * G + q) * 2]));
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float ms = __ldcg(&p.part_ml[((first + s) * G + q) * 2]);
      const float ls = __ldcg(&p.part_ml[((first + s) * G + q) * 2 + 1]);
      const float w = ls > 0.f ? exp2f(ms - M) : 0.f;    // an empty split has l = 0 and m = -inf
      L += ls * w;
      acc += __ldcg(&p.part_o[((first + s) * G + q) * DD + t]) * w;
    }
    p.out[static_cast<int64_t>(b) * p.hq * DD + static_cast<int64_t>(hk * G + q) * DD + t] = __float2bfloat16_rn(acc / L);
  }
  if (t == 0) p.tickets[b * p.hkv + hk] = 0;             // zero again for the next launch
}

// One thread per rotation pair of a query or key head, plus one per 16-byte chunk of a value head.
__global__ void hb_rope_append_kernel(__nv_bfloat16* qkv, __nv_bfloat16* kv, const int32_t* pos_ptr, int batch, int hq,
                                      int hkv, int s_max, int64_t row_stride, double log2_base, int32_t* status) {
  asm volatile("griddepcontrol.wait;\n\tgriddepcontrol.launch_dependents;" ::: "memory");   // see hb_launch_dependent
  const int pos = *pos_ptr;
  if (pos < 0 || pos >= s_max) {                          // cache full: report, write nothing
    if (blockIdx.x == 0 && threadIdx.x == 0 && status) { atomicCAS(status, 0, HB_ERR_INVALID); status[1] = HB_KTAG_DECODE; status[2] = pos; }
    return;
  }
  constexpr int HALF = DD / 2;
  const int n_rot = batch * (hq + hkv) * HALF;
  const int n_val = batch * hkv * (DD / 8);
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < n_rot) {
    const int i = idx % HALF;
    const int head = (idx / HALF) % (hq + hkv);
    const int b = idx / (HALF * (hq + hkv));
    double s, c;
    sincos((double)pos * exp2(-2.0 * i / DD * log2_base), &s, &c);
    const float cf = (float)c, sf = (float)s;
    __nv_bfloat16* h = qkv + b * row_stride + static_cast<int64_t>(head) * DD;   // k heads follow the q heads
    const float a = __bfloat162float(h[i]), bb = __bfloat162float(h[i + HALF]);
    const __nv_bfloat16 lo = __float2bfloat16_rn(a * cf - bb * sf), hi = __float2bfloat16_rn(bb * cf + a * sf);
    h[i] = lo;
    h[i + HALF] = hi;
    if (head >= hq) {
      __nv_bfloat16* dst = kv + ((static_cast<int64_t>(b) * s_max + pos) * hkv + (head - hq)) * DD;
      dst[i] = lo;
      dst[i + HALF] = hi;
    }
  } else if (idx < n_rot + n_val) {
    const int j = idx - n_rot;
    const int c = j % (DD / 8);
    const int hv = (j / (DD / 8)) % hkv;
    const int b = j / ((DD / 8) * hkv);
    const uint4 v = *reinterpret_cast<const uint4*>(qkv + b * row_stride + static_cast<int64_t>(hq + hkv + hv) * DD + c * 8);
    *reinterpret_cast<uint4*>(kv + ((static_cast<int64_t>(batch + b) * s_max + pos) * hkv + hv) * DD + c * 8) = v;
  }
}

__global__ void hb_advance_pos_kernel(int32_t* pos, int32_t n) { *pos += n; }

}  // namespace

extern "C" hb_status hb_rope_append(hb_ctx* ctx, void* qkv, int64_t row_stride, void* kv_cache, const int32_t* pos_dev,
                                    int64_t batch, int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim, int64_t s_max,
                                    float base) {
  if (!ctx) return HB_ERR_INVALID;
  if (!qkv || !kv_cache || !pos_dev) return hb_fail(ctx, HB_ERR_INVALID, "rope_append: null pointer");
  if (batch <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || s_max <= 0) return hb_fail(ctx, HB_ERR_INVALID, "rope_append: empty dimension");
  if (head_dim != DD) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "rope_append: head_dim must be 128");
  if (row_stride < (n_q_heads + 2 * n_kv_heads) * DD || (row_stride & 7))
    return hb_fail(ctx, HB_ERR_INVALID, "rope_append: the row must hold q, k and v heads and be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(kv_cache)) & 15)
    return hb_fail(ctx, HB_ERR_INVALID, "rope_append: pointers must be 16-byte aligned");
  if (!(base > 1.0f)) return hb_fail(ctx, HB_ERR_INVALID, "rope_append: base must exceed 1");
  const int64_t work = batch * (n_q_heads + n_kv_heads) * (DD / 2) + batch * n_kv_heads * (DD / 8);
  if (work > INT32_MAX || 2 * batch * s_max * n_kv_heads * DD > (int64_t(1) << 40))
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "rope_append: problem too large");
  hb_launch_dependent(hb_rope_append_kernel, dim3((unsigned)((work + 255) / 256)), dim3(256), 0, ctx->stream,
      static_cast<__nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(kv_cache), pos_dev, (int)batch, (int)n_q_heads,
      (int)n_kv_heads, (int)s_max, row_stride, log2((double)base), ctx->d_status);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "rope_append launch");
}

extern "C" hb_status hb_attention_decode(hb_ctx* ctx, const void* qkv, int64_t row_stride, const void* kv_cache,
                                         const int32_t* pos_dev, void* out, int64_t batch, int64_t n_q_heads,
                                         int64_t n_kv_heads, int64_t head_dim, int64_t s_max, int64_t len_hint, float scale) {
  if (!ctx) return HB_ERR_INVALID;
  if (!qkv || !kv_cache || !pos_dev || !out) return hb_fail(ctx, HB_ERR_INVALID, "attention_decode: null pointer");
  if (batch <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || s_max <= 0) return hb_fail(ctx, HB_ERR_INVALID, "attention_decode: empty dimension");
  if (head_dim != DD) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "attention_decode: head_dim must be 128");
  if (n_q_heads % n_kv_heads || n_q_heads / n_kv_heads > DEC_MAX_G)
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "attention_decode: query heads must be 1..%d times the KV heads", DEC_MAX_G);
  if (row_stride < n_q_heads * DD) return hb_fail(ctx, HB_ERR_INVALID, "attention_decode: row stride smaller than the query heads");
  if ((reinterpret_cast<uintptr_t>(kv_cache) & 15)) return hb_fail(ctx, HB_ERR_INVALID, "attention_decode: the cache must be 16-byte aligned");
  if (!(scale > 0.f) || !isfinite(scale)) return hb_fail(ctx, HB_ERR_INVALID, "attention_decode: scale must be positive and finite");
  if (batch * n_kv_heads > HB_MAX_SPLITK_TILES || batch > 65535 || n_kv_heads > 65535)
    return hb_fail(ctx, HB_ERR_UNSUPPORTED, "attention_decode: batch * kv_heads exceeds %d", HB_MAX_SPLITK_TILES);
  if (len_hint <= 0 || len_hint > s_max) len_hint = s_max;
  static int resident_per_sm[64] = {};
  if (!resident_per_sm[ctx->device & 63]) {
    cudaError_t e = cudaFuncSetAttribute(hb_attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(DecSmem));
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaFuncSetAttribute(attention_decode)");
    int n = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, hb_attention_decode_kernel, DEC_THREADS, sizeof(DecSmem));
    if (e != cudaSuccess || n < 1) { cudaGetLastError(); n = 1; }
    resident_per_sm[ctx->device & 63] = n;
  }
  // As many splits as fill the GPU ONCE: every CTA streams an equal share of the cache, so a
  // grid that is a little larger than what is resident at one time (512 CTAs on 444 slots)
  // runs a nearly empty second wave and takes twice as long.  Each split is at least one tile.
  const int64_t groups = batch * n_kv_heads;
  const int64_t tiles = (len_hint + DEC_TILE - 1) / DEC_TILE;
  const int64_t slots = (int64_t)ctx->sm_count * resident_per_sm[ctx->device & 63];
  int64_t splits = slots / groups;
  if (splits > tiles) splits = tiles;
  if (splits < 1) splits = 1;
  if (splits > 256) splits = 256;
  // the splits must cover s_max, because the true length is only known on the device
  const int64_t all_tiles = (s_max + DEC_TILE - 1) / DEC_TILE;
  int64_t chunk_tiles = (tiles + splits - 1) / splits;
  splits = (all_tiles + chunk_tiles - 1) / chunk_tiles;
  if (splits > 1024) { chunk_tiles = (all_tiles + 1023) / 1024; splits = (all_tiles + chunk_tiles - 1) / chunk_tiles; }
  const int G = (int)(n_q_heads / n_kv_heads);
  const size_t o_bytes = (size_t)groups * splits * G * DD * sizeof(float);
  const size_t ml_bytes = (size_t)groups * splits * G * 2 * sizeof(float);
  void* ws = nullptr;
  hb_status st = hb_get_scratch(ctx, HB_SCRATCH_DECODE, o_bytes + ml_bytes, &ws);
  if (st != HB_OK) return st;
  DecodeParams p;
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.kv = static_cast<const __nv_bfloat16*>(kv_cache);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = static_cast<float*>(ws);
  p.part_ml = reinterpret_cast<float*>(static_cast<char*>(ws) + o_bytes);
  p.tickets = ctx->d_tickets;
  p.pos = pos_dev;
  p.row_stride = row_stride;
  p.batch = (int)batch; p.hq = (int)n_q_heads; p.hkv = (int)n_kv_heads; p.G = G; p.s_max = (int)s_max;
  p.splits = (int)splits;
  p.chunk = (int)chunk_tiles * DEC_TILE;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = ctx->d_status;
  hb_launch_dependent(hb_attention_decode_kernel, dim3((unsigned)splits, (unsigned)n_kv_heads, (unsigned)batch),
                      dim3(DEC_THREADS), sizeof(DecSmem), ctx->stream, p);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "attention_decode launch");
}

extern "C" hb_status hb_advance_pos(hb_ctx* ctx, int32_t* pos_dev, int32_t n) {
  if (!ctx) return HB_ERR_INVALID;
  if (!pos_dev) return hb_fail(ctx, HB_ERR_INVALID, "advance_pos: null pointer");
  hb_advance_pos_kernel<<<1, 1, 0, ctx->stream>>>(pos_dev, n);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "advance_pos launch");
}
