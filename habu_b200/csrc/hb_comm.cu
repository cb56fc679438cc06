// Collective node: sum-allreduce across the GPUs of one box.
//
//   HB_AR_NCCL  ncclAllReduce enqueued on the context's stream.  NCCL is bound at run time
//               (dlopen of the libnccl.so.2 already in the process, else the system one), so
//               the library neither links NCCL nor pulls a second copy into a host process
//               that already carries one.
//   HB_AR_P2P   this library's two-shot kernel over peer-mapped buffers (NVLink through
//               NVSwitch): every rank owns 1/world of the elements, READS that slice from
//               each peer with plain loads, adds in rank order in fp32, and WRITES the sum
//               into every rank's buffer with plain stores.  Each CTA handshakes only with
//               the same-numbered CTA of the peers (flag words in the symmetric buffer,
//               release/acquire at system scope), so no CTA ever waits on another CTA of its
//               own GPU.  Every wait is bounded: on time-out the kernel records
//               HB_ERR_TIMEOUT and returns.  No multimem and no multicast loads are used.
//   HB_AR_NVLS  the same two phases with the sum taken inside NVSwitch: each rank issues
//               multimem.ld_reduce on the multicast mapping of its slice (the switch reads the
//               slice from every GPU and returns the fp32-accumulated sum) and multimem.st
//               broadcasts the result to every GPU.  Needs a multicast mapping of the
//               symmetric buffer, supplied by the caller through hb_p2p_attach_external.
// Algorithmic bytes per rank: 2 * (world-1)/world * count * elem over NVLink (P2P).
#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>

#include "hb_internal.h"

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
};

NcclApi* nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    const char* env = getenv("HB_NCCL_LIB");
    if (!h && env) h = dlopen(env, RTLD_NOW);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW);
    if (!h) return;
    api.handle = h;
#define HB_SYM(field, name) api.field = reinterpret_cast<decltype(api.field)>(dlsym(h, name))
    HB_SYM(GetUniqueId, "ncclGetUniqueId");
    HB_SYM(CommInitRank, "ncclCommInitRank");
    HB_SYM(CommDestroy, "ncclCommDestroy");
    HB_SYM(CommAbort, "ncclCommAbort");
    HB_SYM(AllReduce, "ncclAllReduce");
    HB_SYM(GetErrorString, "ncclGetErrorString");
    HB_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
#undef HB_SYM
    if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.CommDestroy) api.handle = nullptr;
  });
  return api.handle ? &api : nullptr;
}

// ------------------------------------------------------------------ P2P two-shot kernel
constexpr int AR_MAX_WORLD = 8;
constexpr int AR_MAX_CTAS = 296;                       // 2 per SM on a 148-SM part
constexpr int AR_THREADS = 256;
constexpr size_t AR_HANDSHAKE_BYTES = 2 * AR_MAX_CTAS * AR_MAX_WORLD * sizeof(uint32_t);
// After the per-CTA handshake words: one "rows ready" word per block of gathered rows (written by
// the block's owner into every rank's copy, read by the matmul that consumes the rows) and one
// arrival counter per block (local use: the rows of a block are normalised by different warps).
constexpr int AR_MAX_READY = 512;
constexpr size_t AR_READY_OFF = AR_HANDSHAKE_BYTES;
constexpr size_t AR_COUNT_OFF = AR_READY_OFF + AR_MAX_READY * sizeof(uint32_t);
constexpr size_t AR_FLAG_BYTES = AR_COUNT_OFF + AR_MAX_READY * sizeof(uint32_t);

struct ArParams {
  void* peers[AR_MAX_WORLD];      // base of every rank's symmetric buffer (data first)
  size_t flag_off;                // byte offset of the flag block inside each buffer
  size_t data_off;                // byte offset of the payload inside each buffer
  int64_t count;                  // elements
  int world, rank;
  uint32_t epoch;
  uint32_t spin_limit;            // polls per flag wait before the kernel gives up
  int32_t* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Handshake `phase` (0 start, 1 end) of CTA `cta` with the same CTA on every peer.
__device__ bool ar_barrier(const ArParams& p, int phase, int cta) {
  __threadfence_system();
  __syncthreads();
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const int peer = threadIdx.x;
    // my arrival, written into the peer's flag block at [phase][cta][my rank]
    uint32_t* remote = reinterpret_cast<uint32_t*>(static_cast<char*>(p.peers[peer]) + p.flag_off) +
                       (static_cast<size_t>(phase) * AR_MAX_CTAS + cta) * AR_MAX_WORLD + p.rank;
    st_release_sys(remote, p.epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(static_cast<char*>(p.peers[p.rank]) + p.flag_off) +
                           (static_cast<size_t>(phase) * AR_MAX_CTAS + cta) * AR_MAX_WORLD + peer;
    uint32_t it = 0;
    // epochs only grow; a peer that is already one call ahead has also passed this one
    while (static_cast<int32_t>(ld_acquire_sys(mine) - p.epoch) < 0) {
      if (++it > p.spin_limit) { failed = 1; break; }
    }
  }
  __syncthreads();
  const bool ok = failed == 0;
  if (!ok && threadIdx.x == 0 && p.status) {
    atomicCAS(p.status, 0, HB_ERR_TIMEOUT);
    p.status[1] = HB_KTAG_ALLREDUCE;
    p.status[2] = phase;
  }
  return ok;
}

template <typename T>
struct Vec;   // 16-byte vector of T with fp32 accumulate helpers
template <>
struct Vec<float> {
  static constexpr int N = 4;
  static __device__ void add(float (&acc)[4], const uint4& v) {
    acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
  }
  static __device__ uint4 pack(const float (&acc)[4]) {
    return make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
  }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ void add(float (&acc)[8], const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
      acc[2 * k] += f.x;
      acc[2 * k + 1] += f.y;
    }
  }
  static __device__ uint4 pack(const float (&acc)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
      w[k] = *reinterpret_cast<uint32_t*>(&b);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// WORLD is the unroll bound (2, 4 or 8; other rank counts run the 8-way body with the
// absent ranks predicated off).  256 threads and at most 64 registers, so that a CTA of
// this kernel fits on an SM next to a persistent GEMM CTA when the collective overlaps
// compute on the side stream.
template <typename T, int WORLD>
__global__ void __launch_bounds__(AR_THREADS, 4)
hb_allreduce_p2p_kernel(const ArParams p) {
  constexpr int N = Vec<T>::N;
  const int cta = blockIdx.x;
  if (!ar_barrier(p, 0, cta)) return;
  // Slice owned by this rank, in 16-byte vectors; the tail (count % N) is handled by rank 0.
  const int64_t nvec = p.count / N;
  const int64_t per = (nvec + p.world - 1) / p.world;
  const int64_t v0 = per * p.rank;
  const int64_t v1 = min(nvec, v0 + per);
  for (int64_t i = v0 + cta * (int64_t)AR_THREADS + threadIdx.x; i < v1; i += (int64_t)gridDim.x * AR_THREADS) {
    uint4 v[WORLD];
#pragma unroll
    for (int r = 0; r < WORLD; ++r)
      if (r < p.world)                             // peer loads over NVLink, all in flight
        v[r] = *(reinterpret_cast<const uint4*>(static_cast<const char*>(p.peers[r]) + p.data_off) + i);
    float acc[N] = {};
#pragma unroll
    for (int r = 0; r < WORLD; ++r)
      if (r < p.world) Vec<T>::add(acc, v[r]);      // fixed rank order: identical on every rank
    const uint4 out = Vec<T>::pack(acc);
#pragma unroll
    for (int r = 0; r < WORLD; ++r)
      if (r < p.world) *(reinterpret_cast<uint4*>(static_cast<char*>(p.peers[r]) + p.data_off) + i) = out;
  }
  if (p.rank == 0 && cta == 0 && threadIdx.x < (int)(p.count % N)) {
    const int64_t e = nvec * N + threadIdx.x;
    float s = 0.f;
    for (int r = 0; r < p.world; ++r) {
      const T* q = reinterpret_cast<const T*>(static_cast<char*>(p.peers[r]) + p.data_off);
      s += static_cast<float>(q[e]);
    }
    for (int r = 0; r < p.world; ++r) {
      T* q = reinterpret_cast<T*>(static_cast<char*>(p.peers[r]) + p.data_off);
      q[e] = static_cast<T>(s);
    }
  }
  ar_barrier(p, 1, cta);
}

// ------------------------------------------------------------------ NVLS (in-switch) kernel
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f32(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w) : "memory");
}

// `mc` is the multicast address of the payload.  Same slice ownership and the same
// per-CTA handshakes as the P2P kernel; the element tail (count % N) goes through the
// unicast peer pointers on rank 0.
template <typename T>
__global__ void __launch_bounds__(AR_THREADS, 4)
hb_allreduce_nvls_kernel(const ArParams p, char* mc) {
  constexpr int N = Vec<T>::N;
  const int cta = blockIdx.x;
  if (!ar_barrier(p, 0, cta)) return;
  const int64_t nvec = p.count / N;
  const int64_t per = (nvec + p.world - 1) / p.world;
  const int64_t v0 = per * p.rank;
  const int64_t v1 = min(nvec, v0 + per);
  // Four reductions in flight per thread: a switch round trip is several microseconds, so
  // the bytes in flight, not the SM count, set the rate.
  constexpr int U = 4;
  const int64_t step = (int64_t)gridDim.x * AR_THREADS;
  for (int64_t i = v0 + cta * (int64_t)AR_THREADS + threadIdx.x; i < v1; i += step * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t j = i + u * step;
      if (j < v1) {
        char* a = mc + p.data_off + j * 16;
        v[u] = sizeof(T) == 2 ? multimem_ld_reduce_bf16(a) : multimem_ld_reduce_f32(a);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t j = i + u * step;
      if (j < v1) multimem_st(mc + p.data_off + j * 16, v[u]);
    }
  }
  if (p.rank == 0 && cta == 0 && threadIdx.x < (int)(p.count % N)) {
    const int64_t e = nvec * N + threadIdx.x;
    float s = 0.f;
    for (int r = 0; r < p.world; ++r) s += static_cast<float>(reinterpret_cast<const T*>(static_cast<char*>(p.peers[r]) + p.data_off)[e]);
    for (int r = 0; r < p.world; ++r) reinterpret_cast<T*>(static_cast<char*>(p.peers[r]) + p.data_off)[e] = static_cast<T>(s);
  }
  ar_barrier(p, 1, cta);
}

void comm_kernel_setup(hb_ctx* ctx);   // defined after the fused kernels below

}  // namespace

extern "C" hb_status hb_comm_unique_id(void* id_out) {
  if (!id_out) return HB_ERR_INVALID;
  NcclApi* api = nccl_api();
  if (!api) return HB_ERR_NCCL;
  static_assert(sizeof(ncclUniqueId) <= HB_UNIQUE_ID_BYTES, "unique id size");
  ncclUniqueId id;
  if (api->GetUniqueId(&id) != ncclSuccess) return HB_ERR_NCCL;
  memset(id_out, 0, HB_UNIQUE_ID_BYTES);
  memcpy(id_out, &id, sizeof(id));
  return HB_OK;
}

extern "C" hb_status hb_comm_init_rank(hb_ctx* ctx, int32_t world, int32_t rank, const void* unique_id) {
  if (!ctx) return HB_ERR_INVALID;
  if (world < 1 || rank < 0 || rank >= world) return hb_fail(ctx, HB_ERR_INVALID, "comm: rank %d of %d", rank, world);
  if (ctx->nccl_comm) return hb_fail(ctx, HB_ERR_DUPLICATE, "comm: this context already has a communicator");
  ctx->world = world;
  ctx->rank = rank;
  if (world == 1) return HB_OK;
  if (!unique_id) return hb_fail(ctx, HB_ERR_INVALID, "comm: null unique id");
  NcclApi* api = nccl_api();
  if (!api) return hb_fail(ctx, HB_ERR_NCCL, "comm: libnccl.so.2 could not be loaded");
  cudaError_t ce = cudaSetDevice(ctx->device);
  if (ce != cudaSuccess) return hb_check_cuda(ctx, ce, "cudaSetDevice");
  ncclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  ncclComm_t comm;
  ncclResult_t r = api->CommInitRank(&comm, world, id, rank);
  if (r != ncclSuccess)
    return hb_fail(ctx, HB_ERR_NCCL, "ncclCommInitRank: %s", api->GetErrorString ? api->GetErrorString(r) : "error");
  ctx->nccl_comm = comm;
  return HB_OK;
}

extern "C" hb_status hb_comm_destroy(hb_ctx* ctx) {
  if (!ctx) return HB_ERR_INVALID;
  if (ctx->nccl_comm) {
    NcclApi* api = nccl_api();
    if (api) api->CommDestroy(static_cast<ncclComm_t>(ctx->nccl_comm));
    ctx->nccl_comm = nullptr;
  }
  hb_p2p_state& s = ctx->p2p;
  if (!s.external) {
    for (int r = 0; r < (int)s.peers.size(); ++r)
      if (r != s.rank && s.peers[r]) cudaIpcCloseMemHandle(s.peers[r]);
    if (s.local) cudaFree(s.local);
  }
  s.peers.clear();
  s.local = nullptr;
  s.multicast = nullptr;
  s.external = false;
  s.world = 0;
  return HB_OK;
}

// The symmetric buffer holds `bytes` of payload followed by the flag block.
extern "C" hb_status hb_p2p_alloc(hb_ctx* ctx, size_t bytes, void** dev_ptr, void* handle_out) {
  if (!ctx || !dev_ptr || !handle_out) return HB_ERR_INVALID;
  if (ctx->p2p.local) return hb_fail(ctx, HB_ERR_DUPLICATE, "p2p: this context already owns a symmetric buffer");
  if (bytes == 0) return hb_fail(ctx, HB_ERR_INVALID, "p2p: empty buffer");
  static_assert(sizeof(cudaIpcMemHandle_t) <= HB_IPC_HANDLE_BYTES, "ipc handle size");
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaSetDevice");
  const size_t payload = (bytes + 255) & ~size_t(255);
  void* p = nullptr;
  e = cudaMalloc(&p, payload + AR_FLAG_BYTES);
  if (e != cudaSuccess) { cudaGetLastError(); return hb_fail(ctx, HB_ERR_NOMEM, "p2p: cannot allocate %zu bytes", payload); }
  e = cudaMemset(p, 0, payload + AR_FLAG_BYTES);
  if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaMemset");
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); return hb_check_cuda(ctx, e, "cudaIpcGetMemHandle"); }
  memset(handle_out, 0, HB_IPC_HANDLE_BYTES);
  memcpy(handle_out, &h, sizeof(h));
  ctx->p2p.local = p;
  ctx->p2p.bytes = payload;
  *dev_ptr = p;
  return HB_OK;
}

extern "C" hb_status hb_p2p_attach(hb_ctx* ctx, int32_t world, int32_t rank, const void* all_handles, size_t bytes) {
  if (!ctx || !all_handles) return HB_ERR_INVALID;
  hb_p2p_state& s = ctx->p2p;
  if (!s.local) return hb_fail(ctx, HB_ERR_NOT_FOUND, "p2p: call hb_p2p_alloc first");
  if (world < 1 || world > AR_MAX_WORLD || rank < 0 || rank >= world)
    return hb_fail(ctx, HB_ERR_INVALID, "p2p: rank %d of %d (at most %d ranks)", rank, world, AR_MAX_WORLD);
  if (((bytes + 255) & ~size_t(255)) != s.bytes) return hb_fail(ctx, HB_ERR_INVALID, "p2p: size differs from hb_p2p_alloc");
  if (!s.peers.empty()) return hb_fail(ctx, HB_ERR_DUPLICATE, "p2p: already attached");
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaSetDevice");
  s.peers.assign(world, nullptr);
  for (int r = 0; r < world; ++r) {
    if (r == rank) { s.peers[r] = s.local; continue; }
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const char*>(all_handles) + (size_t)r * HB_IPC_HANDLE_BYTES, sizeof(h));
    e = cudaIpcOpenMemHandle(&s.peers[r], h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      s.peers[r] = nullptr;
      return hb_check_cuda(ctx, e, "cudaIpcOpenMemHandle");
    }
  }
  s.world = world;
  s.rank = rank;
  s.epoch = 0;
  ctx->world = world;
  ctx->rank = rank;
  return HB_OK;
}

extern "C" size_t hb_p2p_flag_bytes(void) { return AR_FLAG_BYTES; }
size_t hb_p2p_ready_offset() { return AR_READY_OFF; }

extern "C" hb_status hb_comm_configure(hb_ctx* ctx, int32_t fused_form, int32_t fused_ctas) {
  if (!ctx) return HB_ERR_INVALID;
  if (fused_form < 0 || fused_form > 2 || fused_ctas < 0)
    return hb_fail(ctx, HB_ERR_INVALID, "comm: fused_form must be 0 (automatic), 1 (CTA per row) or 2 (warp per row)");
  ctx->p2p.fused_form = fused_form;
  ctx->p2p.fused_ctas = fused_ctas;
  return HB_OK;
}

extern "C" hb_status hb_comm_set_wait_limit(hb_ctx* ctx, uint32_t polls) {
  if (!ctx) return HB_ERR_INVALID;
  if (polls == 0) return hb_fail(ctx, HB_ERR_INVALID, "comm: the wait limit must be at least one poll");
  ctx->p2p.spin_limit = polls;
  return HB_OK;
}

// Registers a symmetric buffer the caller allocated and mapped: peer_ptrs[r] is rank r's
// buffer as seen from this process (peer_ptrs[rank] the local one), `multicast_ptr` the
// NVSwitch multicast mapping of the same buffer or NULL.  Each buffer must hold `bytes`
// of payload (rounded up to 256) followed by hb_p2p_flag_bytes() of zeroed flag words.
extern "C" hb_status hb_p2p_attach_external(hb_ctx* ctx, int32_t world, int32_t rank, const void* const* peer_ptrs,
                                            void* multicast_ptr, size_t bytes) {
  if (!ctx || !peer_ptrs) return HB_ERR_INVALID;
  hb_p2p_state& s = ctx->p2p;
  if (s.local) return hb_fail(ctx, HB_ERR_DUPLICATE, "p2p: this context already has a symmetric buffer");
  if (world < 2 || world > AR_MAX_WORLD || rank < 0 || rank >= world)
    return hb_fail(ctx, HB_ERR_INVALID, "p2p: rank %d of %d (2..%d ranks)", rank, world, AR_MAX_WORLD);
  if (bytes == 0) return hb_fail(ctx, HB_ERR_INVALID, "p2p: empty buffer");
  for (int r = 0; r < world; ++r)
    if (!peer_ptrs[r] || (reinterpret_cast<uintptr_t>(peer_ptrs[r]) & 15))
      return hb_fail(ctx, HB_ERR_INVALID, "p2p: peer pointer %d is null or misaligned", r);
  if (reinterpret_cast<uintptr_t>(multicast_ptr) & 15) return hb_fail(ctx, HB_ERR_INVALID, "p2p: misaligned multicast pointer");
  s.peers.assign(world, nullptr);
  for (int r = 0; r < world; ++r) s.peers[r] = const_cast<void*>(peer_ptrs[r]);
  s.local = s.peers[rank];
  s.multicast = multicast_ptr;
  s.external = true;
  s.bytes = (bytes + 255) & ~size_t(255);
  s.world = world;
  s.rank = rank;
  s.epoch = 0;
  ctx->world = world;
  ctx->rank = rank;
  return HB_OK;
}

extern "C" hb_status hb_all_reduce(hb_ctx* ctx, void* data, int64_t count, int32_t dtype, int32_t algo) {
  if (!ctx) return HB_ERR_INVALID;
  if (!data) return hb_fail(ctx, HB_ERR_INVALID, "all_reduce: null pointer");
  if (count <= 0) return hb_fail(ctx, HB_ERR_INVALID, "all_reduce: empty tensor");
  if (dtype != HB_BF16 && dtype != HB_F32) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "all_reduce: dtype %d", dtype);
  if (ctx->world == 1) return HB_OK;   // a single rank already holds the sum
  const size_t es = dtype == HB_BF16 ? 2 : 4;
  hb_p2p_state& s = ctx->p2p;
  const char* lo = static_cast<const char*>(s.local);
  const bool inside = s.world > 1 && static_cast<const char*>(data) >= lo &&
                      static_cast<const char*>(data) + (size_t)count * es <= lo + s.bytes;
  if (algo == HB_AR_AUTO) algo = inside ? (s.multicast ? HB_AR_NVLS : HB_AR_P2P) : HB_AR_NCCL;
  if (algo == HB_AR_NCCL) {
    NcclApi* api = nccl_api();
    if (!api || !ctx->nccl_comm) return hb_fail(ctx, HB_ERR_NCCL, "all_reduce: no NCCL communicator (hb_comm_init_rank)");
    ncclResult_t r = api->AllReduce(data, data, (size_t)count, dtype == HB_BF16 ? ncclBfloat16 : ncclFloat32, ncclSum,
                                    static_cast<ncclComm_t>(ctx->nccl_comm), ctx->stream);
    if (r != ncclSuccess)
      return hb_fail(ctx, HB_ERR_NCCL, "ncclAllReduce: %s", api->GetErrorString ? api->GetErrorString(r) : "error");
    ctx->launches++;
    return HB_OK;
  }
  if (algo != HB_AR_P2P && algo != HB_AR_NVLS) return hb_fail(ctx, HB_ERR_INVALID, "all_reduce: unknown algorithm %d", algo);
  if (algo == HB_AR_NVLS && !s.multicast)
    return hb_fail(ctx, HB_ERR_NOT_FOUND, "all_reduce: no multicast mapping attached (hb_p2p_attach_external)");
  if (s.world < 2) return hb_fail(ctx, HB_ERR_NOT_FOUND, "all_reduce: no peer buffers attached (hb_p2p_attach)");
  if (!inside)
    return hb_fail(ctx, HB_ERR_INVALID, "all_reduce: P2P needs the tensor inside the symmetric buffer of hb_p2p_alloc");
  const size_t off = static_cast<const char*>(data) - lo;
  if (off & 15) return hb_fail(ctx, HB_ERR_INVALID, "all_reduce: tensor must be 16-byte aligned in the symmetric buffer");
  ArParams p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < s.world; ++r) p.peers[r] = s.peers[r];
  p.flag_off = s.bytes;
  p.data_off = off;
  p.count = count;
  p.world = s.world;
  p.rank = s.rank;
  p.epoch = ++s.epoch;
  p.spin_limit = s.spin_limit;
  p.status = ctx->d_status;
  comm_kernel_setup(ctx);
  const int64_t nvec = count / (16 / es);
  int64_t want = (nvec / s.world + AR_THREADS - 1) / AR_THREADS;
  int grid = (int)(want < 1 ? 1 : want);
  int cap = ctx->sm_count * 2 < AR_MAX_CTAS ? ctx->sm_count * 2 : AR_MAX_CTAS;
  if (const char* e = getenv("HB_AR_MAX_CTAS")) {   // every rank must use the same value
    const int v = atoi(e);
    if (v >= 1 && v < cap) cap = v;
  }
  if (grid > cap) grid = cap;
#define HB_AR_LAUNCH(T, W) hb_allreduce_p2p_kernel<T, W><<<grid, AR_THREADS, 0, ctx->stream>>>(p)
  if (algo == HB_AR_NVLS) {
    char* mc = static_cast<char*>(s.multicast);
    if (dtype == HB_BF16) hb_allreduce_nvls_kernel<__nv_bfloat16><<<grid, AR_THREADS, 0, ctx->stream>>>(p, mc);
    else hb_allreduce_nvls_kernel<float><<<grid, AR_THREADS, 0, ctx->stream>>>(p, mc);
  } else if (dtype == HB_BF16) {
    if (s.world == 2) HB_AR_LAUNCH(__nv_bfloat16, 2);
    else if (s.world <= 4) HB_AR_LAUNCH(__nv_bfloat16, 4);
    else HB_AR_LAUNCH(__nv_bfloat16, 8);
  } else {
    if (s.world == 2) HB_AR_LAUNCH(float, 2);
    else if (s.world <= 4) HB_AR_LAUNCH(float, 4);
    else HB_AR_LAUNCH(float, 8);
  }
#undef HB_AR_LAUNCH
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "all_reduce launch");
}

// ---------------------------------------------------------------------------------------
// Fused collective + glue: reduce-scatter -> residual add -> RMSNorm -> all-gather.
//
// After a row-parallel GEMM every rank holds a partial [rows, cols] product.  Instead of
// an allreduce followed by a replicated residual add and RMSNorm on all `rows`, each rank
// owns rows/world rows: it sums the partials of its rows (multimem.ld_reduce through the
// switch, or plain loads from every peer), adds them into its shard of the residual
// stream, normalises, and publishes only the normalised rows to every rank (multimem.st or
// plain peer stores).  NVLink carries the same bytes as the allreduce; the replicated
// elementwise passes disappear and the residual stream stays sharded by rows.
//   mode 0: out[row] = rmsnorm(residual_out[row]) * gain        (published to all ranks)
//   mode 1: out[row] = residual_out[row]                        (final gather of the stream)
// with residual_out[row] = bf16(residual_in[row] + bf16(sum of partials[row])).
// One CTA per row at a time (256 threads, the row in registers), persistent over the
// rank's rows; same per-CTA handshakes and bounded waits as the allreduce kernels.
// ---------------------------------------------------------------------------------------
namespace {

constexpr int ARN_MAX_VEC = 4;   // cols <= 256 * 4 * 8 = 8192 (two rows of operands stay in registers)

struct ArnParams {
  ArParams ar;                 // peers, flag block, world/rank, epoch (data_off = partial's offset)
  size_t out_off;              // byte offset of `out` inside the symmetric buffers
  char* mc;                    // multicast base or null
  const uint4* gain;
  const uint4* residual_in;    // local [rows, cols] (only this rank's rows are read)
  uint4* residual_out;         // local [rows, cols] (only this rank's rows are written)
  int rows, cols8;
  float inv_cols, eps;
  int mode;
  int stagger;                 // rows kernel: pace warps 4..7 behind warps 0..3 (in-switch form)
  int ready_rows;              // rows per "rows ready" word (0: none are published)
};

template <bool NVLS, int WORLD>
__global__ void __launch_bounds__(AR_THREADS, 2)
hb_allreduce_norm_kernel(const ArnParams p) {
  __shared__ float red[AR_THREADS / 32];
  const int cta = blockIdx.x;
  if (!ar_barrier(p.ar, 0, cta)) return;
  const int per = p.rows / p.ar.world;
  const int row0 = per * p.ar.rank;
  // The partial sums of the NEXT row are requested before the current row is normalised,
  // so two rows' worth of switch (or peer) reads are in flight per CTA.
  auto fetch = [&](int row, uint4 (&dst)[ARN_MAX_VEC]) {
    const int64_t base = static_cast<int64_t>(row) * p.cols8;
#pragma unroll
    for (int k = 0; k < ARN_MAX_VEC; ++k) {
      const int c = threadIdx.x + k * AR_THREADS;
      if (c < p.cols8) {
        if (NVLS) {
          dst[k] = multimem_ld_reduce_bf16(p.mc + p.ar.data_off + (base + c) * 16);
        } else {
          uint4 pv[WORLD];
#pragma unroll
          for (int r = 0; r < WORLD; ++r)
            if (r < p.ar.world)
              pv[r] = *(reinterpret_cast<const uint4*>(static_cast<const char*>(p.ar.peers[r]) + p.ar.data_off) + base + c);
          float acc[8] = {};
#pragma unroll
          for (int r = 0; r < WORLD; ++r)
            if (r < p.ar.world) Vec<__nv_bfloat16>::add(acc, pv[r]);
          dst[k] = Vec<__nv_bfloat16>::pack(acc);
        }
      }
    }
  };
  uint4 cur[ARN_MAX_VEC], nxt[ARN_MAX_VEC];
  if (row0 + cta < row0 + per) fetch(row0 + cta, cur);
  for (int row = row0 + cta; row < row0 + per; row += gridDim.x) {
    const int64_t base = static_cast<int64_t>(row) * p.cols8;
    const bool more = row + (int)gridDim.x < row0 + per;
    if (more) fetch(row + gridDim.x, nxt);
    float v[ARN_MAX_VEC][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < ARN_MAX_VEC; ++k) {
      const int c = threadIdx.x + k * AR_THREADS;
      if (c < p.cols8) {
        const uint4 s4 = cur[k];
        const uint4 r4 = p.residual_in[base + c];
        const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w}, rw[4] = {r4.x, r4.y, r4.z, r4.w};
        uint32_t xw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&sw[j]));
          const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rw[j]));
          __nv_bfloat162 x = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
          xw[j] = *reinterpret_cast<uint32_t*>(&x);
          const float2 xf = __bfloat1622float2(x);
          v[k][2 * j] = xf.x;
          v[k][2 * j + 1] = xf.y;
          ss += xf.x * xf.x + xf.y * xf.y;
        }
        p.residual_out[base + c] = make_uint4(xw[0], xw[1], xw[2], xw[3]);
      }
    }
    float inv = 1.0f;
    if (p.mode == 0) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      __syncthreads();                         // red[] from the previous row has been read
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < AR_THREADS / 32; ++w) tot += red[w];
      inv = rsqrtf(tot * p.inv_cols + p.eps);
    }
#pragma unroll
    for (int k = 0; k < ARN_MAX_VEC; ++k) {
      const int c = threadIdx.x + k * AR_THREADS;
      if (c < p.cols8) {
        uint32_t o[4];
        if (p.mode == 0) {
          const uint4 g = __ldg(p.gain + c);
          const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[j]));
            __nv_bfloat162 h = __floats2bfloat162_rn(v[k][2 * j] * inv * gf.x, v[k][2 * j + 1] * inv * gf.y);
            o[j] = *reinterpret_cast<uint32_t*>(&h);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[k][2 * j], v[k][2 * j + 1]);
            o[j] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        const uint4 o4 = make_uint4(o[0], o[1], o[2], o[3]);
        if (NVLS) {
          multimem_st(p.mc + p.out_off + (base + c) * 16, o4);
        } else {
#pragma unroll
          for (int r = 0; r < WORLD; ++r)
            if (r < p.ar.world) *(reinterpret_cast<uint4*>(static_cast<char*>(p.ar.peers[r]) + p.out_off) + base + c) = o4;
        }
      }
    }
    if (more) {
#pragma unroll
      for (int k = 0; k < ARN_MAX_VEC; ++k) cur[k] = nxt[k];
    }
  }
  ar_barrier(p.ar, 1, cta);
}


// Warp-per-row form of the same kernel for cols <= 4096 (the decoder's width).  A CTA-wide
// barrier per row kept only two rows (16 KB) in flight per CTA; a switch or peer round trip is
// several microseconds, so the kernel ran at less than half the NVLink rate.  Here every warp
// owns whole rows: its 32 lanes hold the row (up to 16 x 16 B per lane), reduce the sum of
// squares with shuffles only, and the eight warps of a CTA work on eight different rows at
// different phases, so loads of some rows overlap the stores of others with no barrier between
// them.  Few CTAs are needed (rows / 8 at most), which leaves the SMs to a GEMM that runs
// beside it.  The arithmetic and its order are those of the CTA-per-row kernel and of
// rmsnorm_kernel (lane l of virtual warp w sums vectors c = 32 (w + 8 k) + l, k = 0..3; then
// the shuffle tree; then the eight warp sums in order), so the results are the same bits.
constexpr int ARW_VEC = 16;    // 16-byte vectors per lane: cols <= 32 * 16 * 8 = 4096
constexpr int ARW_ROUNDS = 64; // most rounds (rows per warp) when ready words are published

template <bool NVLS, int WORLD>
__global__ void __launch_bounds__(AR_THREADS, 2)
hb_allreduce_norm_rows_kernel(const ArnParams p) {
  // Pacing between the two halves of the CTA (see `stagger` below).
  __shared__ volatile int loaded[AR_THREADS / 64];
  __shared__ int round_rows[ARW_ROUNDS];       // rows of this CTA done per round (ready words)
  const int cta = blockIdx.x;
  if (threadIdx.x < AR_THREADS / 64) loaded[threadIdx.x] = 0;
  if (threadIdx.x < ARW_ROUNDS) round_rows[threadIdx.x] = 0;
  if (!ar_barrier(p.ar, 0, cta)) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per = p.rows / p.ar.world;
  const int row0 = per * p.ar.rank;
  const int nwarps = gridDim.x * (AR_THREADS / 32);
  // In the in-switch form the two phases of a row load opposite directions of the link: the
  // reduction pulls every rank's copy of the row through this GPU's outgoing lanes (world x the
  // bytes it receives), the broadcast store fans out into every GPU's incoming lanes.  Warps that
  // all read and then all write use one direction at a time.  With `stagger` warps 4..7 start a
  // row's reads only when their partner (warp - 4) has received the reads of the same round, so
  // one half of the CTA reads while the other half writes.  The pacing is a hint, not a
  // dependency: a wait that runs out simply proceeds.
  const bool follower = p.stagger && warp >= AR_THREADS / 64;
  const int pair_slot = warp & (AR_THREADS / 64 - 1);
  int round = 0;
  for (int row = row0 + cta * (AR_THREADS / 32) + warp; row < row0 + per; row += nwarps, ++round) {
    const int64_t base = static_cast<int64_t>(row) * p.cols8;
    uint4 s[ARW_VEC];
    if (follower) {
      if (lane == 0) {
        for (int it = 0; loaded[pair_slot] <= round && it < (1 << 16); ++it) __nanosleep(64);
      }
      __syncwarp();
    }
    if (NVLS) {
#pragma unroll
      for (int k = 0; k < ARW_VEC; ++k) {
        const int c = lane + 32 * k;
        if (c < p.cols8) s[k] = multimem_ld_reduce_bf16(p.mc + p.ar.data_off + (base + c) * 16);
      }
    } else {
#pragma unroll
      for (int k = 0; k < ARW_VEC; ++k) {
        const int c = lane + 32 * k;
        if (c < p.cols8) {
          uint4 pv[WORLD];
#pragma unroll
          for (int r = 0; r < WORLD; ++r)
            if (r < p.ar.world)
              pv[r] = *(reinterpret_cast<const uint4*>(static_cast<const char*>(p.ar.peers[r]) + p.ar.data_off) + base + c);
          float acc[8] = {};
#pragma unroll
          for (int r = 0; r < WORLD; ++r)
            if (r < p.ar.world) Vec<__nv_bfloat16>::add(acc, pv[r]);
          s[k] = Vec<__nv_bfloat16>::pack(acc);
        }
      }
    }
    // residual add (rounded to bf16, which is what gets normalised) and the sums of squares,
    // one partial sum per virtual warp w = k % 8
    float ssw[8] = {};
#pragma unroll
    for (int k = 0; k < ARW_VEC; ++k) {
      const int c = lane + 32 * k;
      if (c < p.cols8) {
        const uint4 r4 = p.residual_in[base + c];
        const uint32_t sw[4] = {s[k].x, s[k].y, s[k].z, s[k].w}, rw[4] = {r4.x, r4.y, r4.z, r4.w};
        uint32_t xw[4];
        float ss = ssw[k & 7];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&sw[j]));
          const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rw[j]));
          __nv_bfloat162 x = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
          xw[j] = *reinterpret_cast<uint32_t*>(&x);
          const float2 xf = __bfloat1622float2(x);
          ss += xf.x * xf.x + xf.y * xf.y;
        }
        ssw[k & 7] = ss;
        s[k] = make_uint4(xw[0], xw[1], xw[2], xw[3]);
        p.residual_out[base + c] = s[k];
      }
    }
    if (p.stagger && !follower && lane == 0) loaded[pair_slot] = round + 1;   // this round's reads have landed
    float inv = 1.0f;
    if (p.mode == 0) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        float v = ssw[w];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        tot += v;
      }
      inv = rsqrtf(tot * p.inv_cols + p.eps);
    }
#pragma unroll
    for (int k = 0; k < ARW_VEC; ++k) {
      const int c = lane + 32 * k;
      if (c < p.cols8) {
        uint4 o4 = s[k];
        if (p.mode == 0) {
          const uint4 g = __ldg(p.gain + c);
          const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, xw[4] = {s[k].x, s[k].y, s[k].z, s[k].w};
          uint32_t o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[j]));
            const float2 xf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xw[j]));
            __nv_bfloat162 h = __floats2bfloat162_rn(xf.x * inv * gf.x, xf.y * inv * gf.y);
            o[j] = *reinterpret_cast<uint32_t*>(&h);
          }
          o4 = make_uint4(o[0], o[1], o[2], o[3]);
        }
        if (NVLS) {
          multimem_st(p.mc + p.out_off + (base + c) * 16, o4);
        } else {
#pragma unroll
          for (int r = 0; r < WORLD; ++r)
            if (r < p.ar.world) *(reinterpret_cast<uint4*>(static_cast<char*>(p.ar.peers[r]) + p.out_off) + base + c) = o4;
        }
      }
    }
    if (p.ready_rows) {
      // "Rows ready" words: a matmul that consumes the gathered rows waits for the word of a
      // block of rows instead of for the end of this kernel.  A system-scope fence is costly
      // (it waits for the SM's stores in flight), so there is one per CTA and round, not one per
      // row: the eight rows a CTA handles in a round lie in one block; each warp counts its row
      // in shared memory, and the warp that completes the CTA's share fences once, adds the
      // share to the block's counter, and, if that completes the block, writes the word into
      // every rank's copy.  Only that one warp waits; the others go on to their next rows.
      __syncwarp();
      if (lane == 0) {
        const int first = row0 + round * nwarps + cta * (AR_THREADS / 32);   // the CTA's first row of this round
        const int share = min(AR_THREADS / 32, row0 + per - first);
        __threadfence_block();
        if (atomicAdd(&round_rows[round & (ARW_ROUNDS - 1)], 1) == share - 1) {
          round_rows[round & (ARW_ROUNDS - 1)] = 0;
          __threadfence_system();                     // the CTA's rows of this round, before the count
          const int blk = first / p.ready_rows;
          char* mine = static_cast<char*>(p.ar.peers[p.ar.rank]) + p.ar.flag_off;
          int* count = reinterpret_cast<int*>(mine + AR_COUNT_OFF) + blk;
          if (atomicAdd(count, share) == p.ready_rows - share) {
            *count = 0;                               // zero again for the next launch
            __threadfence_system();                   // the other CTAs' rows, before the word
            for (int r = 0; r < p.ar.world; ++r)
              st_release_sys(reinterpret_cast<uint32_t*>(static_cast<char*>(p.ar.peers[r]) + p.ar.flag_off + AR_READY_OFF) + blk,
                             p.ar.epoch);
          }
        }
      }
    }
  }
  if (p.stagger && !follower && lane == 0) loaded[pair_slot] = 1 << 30;   // no more rounds: followers run free
  ar_barrier(p.ar, 1, cta);
}

// The collective kernels use almost no shared memory, the GEMM and attention kernels they
// run beside use nearly all of it.  An SM holds CTAs of two kernels at the same time only if
// both were launched with the same split between L1 and shared memory, so the collective
// kernels ask for the largest shared-memory carve-out too (HB_AR_CARVEOUT=0 leaves the
// driver's choice).
template <typename K>
void set_carveout(K kernel, int value) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, value);
}
void comm_kernel_setup(hb_ctx* ctx) {
  static int applied[64];
  static bool init = false;
  if (!init) { for (int& a : applied) a = -2; init = true; }
  int want = cudaSharedmemCarveoutMaxShared;
  if (const char* e = getenv("HB_AR_CARVEOUT"))
    if (atoi(e) == 0) want = cudaSharedmemCarveoutDefault;
  if (applied[ctx->device & 63] == want) return;
  applied[ctx->device & 63] = want;
  set_carveout(hb_allreduce_p2p_kernel<float, 2>, want); set_carveout(hb_allreduce_p2p_kernel<float, 4>, want);
  set_carveout(hb_allreduce_p2p_kernel<float, 8>, want); set_carveout(hb_allreduce_p2p_kernel<__nv_bfloat16, 2>, want);
  set_carveout(hb_allreduce_p2p_kernel<__nv_bfloat16, 4>, want); set_carveout(hb_allreduce_p2p_kernel<__nv_bfloat16, 8>, want);
  set_carveout(hb_allreduce_nvls_kernel<float>, want); set_carveout(hb_allreduce_nvls_kernel<__nv_bfloat16>, want);
  set_carveout(hb_allreduce_norm_kernel<true, 1>, want); set_carveout(hb_allreduce_norm_kernel<false, 2>, want);
  set_carveout(hb_allreduce_norm_kernel<false, 4>, want); set_carveout(hb_allreduce_norm_kernel<false, 8>, want);
  set_carveout(hb_allreduce_norm_rows_kernel<true, 1>, want); set_carveout(hb_allreduce_norm_rows_kernel<false, 2>, want);
  set_carveout(hb_allreduce_norm_rows_kernel<false, 4>, want); set_carveout(hb_allreduce_norm_rows_kernel<false, 8>, want);
  cudaGetLastError();
}

}  // namespace

extern "C" hb_status hb_all_reduce_norm(hb_ctx* ctx, const void* partial, const void* gain, const void* residual_in,
                                        void* residual_out, void* out, int64_t rows, int64_t cols, float eps,
                                        int32_t mode, int32_t algo) {
  if (!ctx) return HB_ERR_INVALID;
  if (!partial || !residual_in || !residual_out || !out || (mode == 0 && !gain))
    return hb_fail(ctx, HB_ERR_INVALID, "all_reduce_norm: null pointer");
  const bool publish = (mode & 2) != 0;      // publish "rows ready" words for hb_matmul_gathered
  mode &= ~2;
  if (mode != 0 && mode != 1) return hb_fail(ctx, HB_ERR_INVALID, "all_reduce_norm: unknown mode %d", mode);
  hb_p2p_state& s = ctx->p2p;
  if (s.world < 2) return hb_fail(ctx, HB_ERR_NOT_FOUND, "all_reduce_norm: no peer buffers attached");
  if (rows <= 0 || cols <= 0 || rows % s.world) return hb_fail(ctx, HB_ERR_INVALID, "all_reduce_norm: rows must split evenly over the ranks");
  if (cols % 8 || cols > AR_THREADS * ARN_MAX_VEC * 8) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "all_reduce_norm: cols must be a multiple of 8, at most %d", AR_THREADS * ARN_MAX_VEC * 8);
  const char* lo = static_cast<const char*>(s.local);
  const size_t nbytes = (size_t)rows * cols * 2;
  auto inside = [&](const void* p) { return static_cast<const char*>(p) >= lo && static_cast<const char*>(p) + nbytes <= lo + s.bytes; };
  if (!inside(partial) || !inside(out)) return hb_fail(ctx, HB_ERR_INVALID, "all_reduce_norm: partial and out must lie in the symmetric buffer");
  if ((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(gain) |
       reinterpret_cast<uintptr_t>(residual_in) | reinterpret_cast<uintptr_t>(residual_out)) & 15)
    return hb_fail(ctx, HB_ERR_INVALID, "all_reduce_norm: pointers must be 16-byte aligned");
  if (algo == HB_AR_AUTO) algo = s.multicast ? HB_AR_NVLS : HB_AR_P2P;
  if (algo == HB_AR_NVLS && !s.multicast) return hb_fail(ctx, HB_ERR_NOT_FOUND, "all_reduce_norm: no multicast mapping attached");
  if (algo != HB_AR_NVLS && algo != HB_AR_P2P) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "all_reduce_norm: algorithm %d", algo);
  ArnParams p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < s.world; ++r) p.ar.peers[r] = s.peers[r];
  p.ar.flag_off = s.bytes;
  p.ar.data_off = static_cast<const char*>(partial) - lo;
  p.ar.count = rows * cols;
  p.ar.world = s.world;
  p.ar.rank = s.rank;
  p.ar.epoch = ++s.epoch;
  p.ar.spin_limit = s.spin_limit;
  p.ar.status = ctx->d_status;
  p.out_off = static_cast<const char*>(out) - lo;
  p.mc = static_cast<char*>(s.multicast);
  p.gain = static_cast<const uint4*>(gain);
  p.residual_in = static_cast<const uint4*>(residual_in);
  p.residual_out = static_cast<uint4*>(residual_out);
  p.rows = (int)rows;
  p.cols8 = (int)(cols / 8);
  p.inv_cols = 1.0f / (float)cols;
  p.eps = eps;
  p.mode = mode;
  comm_kernel_setup(ctx);
  // Two forms of the kernel.  One CTA per row (two rows in flight per CTA, up to two CTAs per
  // SM) is the faster one when the collective has the GPU to itself: measured 194 us against
  // 233 us for a 64 MiB exchange over 8 GPUs.  One warp per row needs few CTAs and at most 128
  // registers, which is what lets it run beside a GEMM on the same SMs: the form for
  // collectives that overlap compute.  hb_comm_configure chooses; the default is the CTA-per-row
  // form on the context's own stream and the warp-per-row form on the side stream.
  int form = s.fused_form;
  if (form == 0) form = (ctx->stream == ctx->side_stream && ctx->side_stream) ? 2 : 1;
  if (const char* e = getenv("HB_ARN_ROWS")) form = atoi(e) != 0 ? 2 : 1;
  if (publish) form = 2;                               // only the warp-per-row form publishes ready words
  const bool by_rows = form == 2 && cols <= 32 * ARW_VEC * 8;
  const int per = (int)(rows / s.world);
  s.ready_rows = 0;
  p.ready_rows = 0;
  if (by_rows) {
    int grid = (per + AR_THREADS / 32 - 1) / (AR_THREADS / 32);
    int cap = ctx->sm_count < AR_MAX_CTAS ? ctx->sm_count : AR_MAX_CTAS;
    if (s.fused_ctas >= 1 && s.fused_ctas < cap) cap = s.fused_ctas;
    if (const char* e = getenv("HB_ARN_CTAS")) {      // every rank must use the same value
      const int v = atoi(e);
      if (v >= 1 && v < cap) cap = v;
    } else if (const char* e = getenv("HB_AR_MAX_CTAS")) {
      const int v = atoi(e);
      if (v >= 1 && v < cap) cap = v;
    }
    if (grid > cap) grid = cap;
    p.stagger = algo == HB_AR_NVLS ? 1 : 0;
    if (const char* e = getenv("HB_ARN_STAGGER")) p.stagger = atoi(e) != 0;
    if (publish) {
      // rows per ready word: at most 256 (a matmul row tile), a multiple of the eight rows a CTA
      // handles per round, dividing every rank's share
      int rb = per >= 256 ? 256 : per;
      while (rb > 8 && per % rb) rb >>= 1;
      const int rounds = (per + grid * (AR_THREADS / 32) - 1) / (grid * (AR_THREADS / 32));
      if (rb % (AR_THREADS / 32) == 0 && per % rb == 0 && rows / rb <= AR_MAX_READY && rounds <= ARW_ROUNDS) {
        p.ready_rows = rb;
        s.ready_rows = rb;
        s.ready_epoch = p.ar.epoch;
        s.ready_out = out;
        s.ready_total_rows = rows;
      }
    }
    if (algo == HB_AR_NVLS) hb_allreduce_norm_rows_kernel<true, 1><<<grid, AR_THREADS, 0, ctx->stream>>>(p);
    else if (s.world == 2) hb_allreduce_norm_rows_kernel<false, 2><<<grid, AR_THREADS, 0, ctx->stream>>>(p);
    else if (s.world <= 4) hb_allreduce_norm_rows_kernel<false, 4><<<grid, AR_THREADS, 0, ctx->stream>>>(p);
    else hb_allreduce_norm_rows_kernel<false, 8><<<grid, AR_THREADS, 0, ctx->stream>>>(p);
    ctx->launches++;
    return hb_check_cuda(ctx, cudaGetLastError(), "all_reduce_norm launch");
  }
  int grid = (int)(rows / s.world);
  int cap = ctx->sm_count * 2 < AR_MAX_CTAS ? ctx->sm_count * 2 : AR_MAX_CTAS;
  if (grid > cap) grid = cap;
  if (algo == HB_AR_NVLS) hb_allreduce_norm_kernel<true, 1><<<grid, AR_THREADS, 0, ctx->stream>>>(p);
  else if (s.world == 2) hb_allreduce_norm_kernel<false, 2><<<grid, AR_THREADS, 0, ctx->stream>>>(p);
  else if (s.world <= 4) hb_allreduce_norm_kernel<false, 4><<<grid, AR_THREADS, 0, ctx->stream>>>(p);
  else hb_allreduce_norm_kernel<false, 8><<<grid, AR_THREADS, 0, ctx->stream>>>(p);
  ctx->launches++;
  return hb_check_cuda(ctx, cudaGetLastError(), "all_reduce_norm launch");
}

// ---------------------------------------------------------------------------------------
// Overlapped collectives outside the graph executor (the data-parallel trainer): the
// allreduce is enqueued on the context's high-priority side stream, ordered after
// everything already queued on the main stream; hb_side_join makes the main stream wait
// for the side stream.  Between the two calls the main stream is free to run the kernels
// that do not touch the reduced tensor (the rest of the backward pass).
// ---------------------------------------------------------------------------------------
static hb_status ensure_side_stream(hb_ctx* ctx) {
  if (!ctx->side_stream) {
    int lo = 0, hi = 0;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);
    cudaError_t e = cudaStreamCreateWithPriority(&ctx->side_stream, cudaStreamNonBlocking, hi);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaStreamCreate(side)");
  }
  if (!ctx->side_event) {
    cudaError_t e = cudaEventCreateWithFlags(&ctx->side_event, cudaEventDisableTiming);
    if (e != cudaSuccess) return hb_check_cuda(ctx, e, "cudaEventCreate(side)");
  }
  return HB_OK;
}

extern "C" hb_status hb_all_reduce_async(hb_ctx* ctx, void* data, int64_t count, int32_t dtype, int32_t algo) {
  if (!ctx) return HB_ERR_INVALID;
  if (ctx->world == 1) return HB_OK;
  hb_status st = ensure_side_stream(ctx);
  if (st != HB_OK) return st;
  cudaStream_t main_stream = ctx->stream;
  cudaError_t e = cudaEventRecord(ctx->side_event, main_stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->side_stream, ctx->side_event, 0);
  if (e != cudaSuccess) return hb_check_cuda(ctx, e, "all_reduce_async: fork");
  ctx->stream = ctx->side_stream;
  st = hb_all_reduce(ctx, data, count, dtype, algo);
  ctx->stream = main_stream;
  return st;
}

extern "C" hb_status hb_side_join(hb_ctx* ctx) {
  if (!ctx) return HB_ERR_INVALID;
  if (!ctx->side_stream || !ctx->side_event) return HB_OK;
  cudaError_t e = cudaEventRecord(ctx->side_event, ctx->side_stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->stream, ctx->side_event, 0);
  return hb_check_cuda(ctx, e, "side_join");
}
