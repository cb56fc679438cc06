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
constexpr int DEC_TILE = 64;       // cached positions per shared-memory tile
constexpr int DEC_THREADS = 128;
constexpr int DEC_MAX_G = 8;       // query heads per KV head
constexpr int K_ROW = DD + 8;      // bf16 per K row in shared memory (272 B: conflict-free 16-byte reads down a column)

struct DecodeParams {
  const __nv_bfloat16* qkv;        // [batch, row_stride]: q heads, then k heads, then v heads of the new token
  const __nv_bfloat16* kv;         // cache
  __nv_bfloat16* out;              // [batch, hq * 128]
  float* part_o;                   // [batch * hkv * splits * G][128]
  float* part_ml;                  // [batch * hkv * splits * G][2]  (running max in log2 units, sum)
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

struct DecSmem {
  __nv_bfloat16 k[2][DEC_TILE][K_ROW];
  __nv_bfloat16 v[2][DEC_TILE][DD];
  float q[DEC_MAX_G][DD];          // queries, pre-multiplied by scale * log2(e)
  float p[DEC_TILE][DEC_MAX_G];    // scores, then probabilities, of the current tile
  float alpha[DEC_MAX_G], m[DEC_MAX_G], l[DEC_MAX_G];
  int last;
};

__global__ void __launch_bounds__(DEC_THREADS)
hb_attention_decode_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) uint8_t dec_smem_raw[];
  DecSmem& sm = *reinterpret_cast<DecSmem*>(dec_smem_raw);
  // the attention-out product behind this kernel may start streaming its weights in
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int G = p.G;
  int len = *p.pos + 1;
  if (len > p.s_max) len = p.s_max;        // the append kernel has already reported the overflow
  const int begin = split * p.chunk;
  const int end = min(begin + p.chunk, len);
  const int64_t slot = (static_cast<int64_t>(b) * p.hkv + hk) * p.splits + split;

  float o[DEC_MAX_G];
#pragma unroll
  for (int q = 0; q < DEC_MAX_G; ++q) o[q] = 0.f;
  if (t < DEC_MAX_G) { sm.m[t] = -INFINITY; sm.l[t] = 0.f; sm.alpha[t] = 1.f; }

  if (begin < end) {
    // queries of this KV head's group -> shared memory, scaled
    for (int i = t; i < G * DD; i += DEC_THREADS) {
      const int q = i / DD, d = i - q * DD;
      sm.q[q][d] = __bfloat162float(p.qkv[b * p.row_stride + static_cast<int64_t>(hk * G + q) * DD + d]) * p.scale_log2;
    }
    const __nv_bfloat16* kbase = p.kv + (static_cast<int64_t>(b) * p.s_max * p.hkv + hk) * DD;
    const __nv_bfloat16* vbase = p.kv + (static_cast<int64_t>(p.batch + b) * p.s_max * p.hkv + hk) * DD;
    const int64_t pos_stride = static_cast<int64_t>(p.hkv) * DD;
    const int n_tiles = (end - begin + DEC_TILE - 1) / DEC_TILE;
    auto load_tile = [&](int tile, int buf) {
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
      cp_async_commit();
    };
    load_tile(0, 0);
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int buf = tile & 1;
      if (tile + 1 < n_tiles) { load_tile(tile + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
      __syncthreads();                                   // tile `buf` (and, first time, q) visible to all
      // ---- scores: thread = (position r, query parity)
      {
        const int r = t & (DEC_TILE - 1), par = t >> 6;
        float acc[DEC_MAX_G / 2];
#pragma unroll
        for (int j = 0; j < DEC_MAX_G / 2; ++j) acc[j] = 0.f;
#pragma unroll 4
        for (int c = 0; c < DD / 8; ++c) {
          const uint4 k8 = *reinterpret_cast<const uint4*>(&sm.k[buf][r][c * 8]);
          const uint32_t kw[4] = {k8.x, k8.y, k8.z, k8.w};
          float kf[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kw[j]));
            kf[2 * j] = f.x; kf[2 * j + 1] = f.y;
          }
#pragma unroll
          for (int j = 0; j < DEC_MAX_G / 2; ++j) {
            const int q = par + 2 * j;
            if (q < G) {
              const float4 q0 = *reinterpret_cast<const float4*>(&sm.q[q][c * 8]);
              const float4 q1 = *reinterpret_cast<const float4*>(&sm.q[q][c * 8 + 4]);
              acc[j] += kf[0] * q0.x + kf[1] * q0.y + kf[2] * q0.z + kf[3] * q0.w + kf[4] * q1.x + kf[5] * q1.y +
                        kf[6] * q1.z + kf[7] * q1.w;
            }
          }
        }
        const bool valid = begin + tile * DEC_TILE + r < end;
#pragma unroll
        for (int j = 0; j < DEC_MAX_G / 2; ++j) {
          const int q = par + 2 * j;
          if (q < G) sm.p[r][q] = valid ? acc[j] : -INFINITY;
        }
      }
      __syncthreads();
      // ---- online softmax: warp w owns queries w and w + 4
      for (int q = warp; q < G; q += DEC_THREADS / 32) {
        const float s0 = sm.p[lane][q], s1 = sm.p[lane + 32][q];
        float mx = fmaxf(s0, s1);
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
        const float m_old = sm.m[q];
        const float m_new = fmaxf(m_old, mx);            // finite: every tile holds a valid position
        const float p0 = exp2f(s0 - m_new), p1 = exp2f(s1 - m_new);
        float sum = p0 + p1;
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o2);
        sm.p[lane][q] = p0;
        sm.p[lane + 32][q] = p1;
        if (lane == 0) {
          const float a = exp2f(m_old - m_new);          // 0 on the first tile (m_old = -inf)
          sm.alpha[q] = a;
          sm.l[q] = sm.l[q] * a + sum;
          sm.m[q] = m_new;
        }
      }
      __syncthreads();
      // ---- O += P V: thread = output dimension d
      {
#pragma unroll
        for (int q = 0; q < DEC_MAX_G; ++q)
          if (q < G) o[q] *= sm.alpha[q];
#pragma unroll 8
        for (int r = 0; r < DEC_TILE; ++r) {
          const float v = __bfloat162float(sm.v[buf][r][t]);
          const float4 pa = *reinterpret_cast<const float4*>(&sm.p[r][0]);
          const float4 pb = *reinterpret_cast<const float4*>(&sm.p[r][4]);
          const float pr[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
          for (int q = 0; q < DEC_MAX_G; ++q)
            if (q < G) o[q] += pr[q] * v;
        }
      }
      __syncthreads();                                   // tile `buf` and p[] are free again
    }
  }
  // ---- this split's partial result
  for (int q = 0; q < G; ++q) p.part_o[(slot * G + q) * DD + t] = o[q];
  if (t < G) {
    p.part_ml[(slot * G + t) * 2] = sm.m[t];
    p.part_ml[(slot * G + t) * 2 + 1] = sm.l[t];
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
  hb_rope_append_kernel<<<(unsigned)((work + 255) / 256), 256, 0, ctx->stream>>>(
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
  hb_attention_decode_kernel<<<dim3((unsigned)splits, (unsigned)n_kv_heads, (unsigned)batch), DEC_THREADS, sizeof(DecSmem),
                               ctx->stream>>>(p);
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
