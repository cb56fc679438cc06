// Internal (non-ABI) declarations shared by the translation units of libhabu_b200.so.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/habu_b200.h"

// Device status word layout (int32[4]): [0] first error code, [1] kernel tag that
// reported it, [2] detail (e.g. which wait), [3] reserved.
enum { HB_KTAG_GEMM = 1, HB_KTAG_ATTN = 2, HB_KTAG_ALLREDUCE = 3, HB_KTAG_SPLITK = 4, HB_KTAG_DECODE = 5 };

// Scratch slots: kernel workspace (split-K partials), host-call staging, autotune operands.
enum { HB_SCRATCH_WORKSPACE = 0, HB_SCRATCH_STAGING = 1, HB_SCRATCH_TUNE = 2, HB_SCRATCH_REDUCE = 3, HB_SCRATCH_DECODE = 4, HB_NUM_SCRATCH = 5 };

constexpr int HB_MAX_SPLITK_TILES = 4096;

struct hb_tune_entry {
  int32_t config_id;   // matmul: index in the configuration table; attention: 0 one unit per CTA, 1 persistent
  float ms;
  int32_t p0, p1;      // stream-K matmul: grid, k-blocks per ring stage
};
enum { HB_OP_SKINNY = 2 };   // cache lines of the stream-K kernel (reached through HB_OP_MATMUL with M <= 64)

// One encoded TMA descriptor and the arguments it was encoded from (see hb_make_tensor_map).
struct hb_tmap_entry {
  alignas(8) unsigned char key[128];
  alignas(64) unsigned char map[128];
};

struct hb_p2p_state {
  int world = 0, rank = 0;
  size_t bytes = 0;
  void* local = nullptr;              // this rank's symmetric buffer (data + flags)
  std::vector<void*> peers;           // mapped base pointers, peers[rank] == local
  void** d_peers = nullptr;           // device copy of `peers`
  void* multicast = nullptr;          // NVSwitch multicast mapping of the same buffer (optional)
  bool external = false;              // buffer and mappings are owned by the caller
  uint32_t epoch = 0;
  uint32_t spin_limit = 1u << 24;     // polls per cross-GPU flag wait before HB_ERR_TIMEOUT
  // "rows ready" words of the last hb_all_reduce_norm (see hb_matmul_gathered): rows per word
  // (0: none), the epoch they carry, the gathered tensor they describe and its row count
  int fused_form = 0, fused_ctas = 0; // hb_comm_configure: kernel form of the fused collective, CTA cap of the warp-per-row form
  int ready_rows = 0;
  uint32_t ready_epoch = 0;
  const void* ready_out = nullptr;
  int64_t ready_total_rows = 0;
};
// Byte offset of the ready words inside the flag block that follows the payload.
size_t hb_p2p_ready_offset();

struct hb_ctx {
  int device = 0;
  int sm_count = 0;
  std::string gpu_name;               // device name with blanks replaced by '_' (part of the autotune key)
  cudaStream_t stream = nullptr;      // stream in use
  cudaStream_t own_stream = nullptr;  // created by the context
  cudaStream_t side_stream = nullptr; // second stream for executor nodes that overlap (collectives)
  cudaEvent_t side_event = nullptr;   // fork / join marker between the two streams
  // host-buffer entry points: copy-in and copy-out streams and a pool of ordering events, so
  // that PCIe transfers in both directions overlap the kernels chunk by chunk
  cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
  std::vector<cudaEvent_t> event_pool;
  int32_t* d_status = nullptr;
  uint32_t attn_launches = 0;   // picks one of the attention work counters kept behind the status words
  int32_t* h_status = nullptr;        // pinned
  int* d_tickets = nullptr;           // split-K arrival tickets, one per output tile, zero between launches
  int64_t launches = 0;
  std::string err;
  std::map<std::string, hb_tune_entry> tune_cache;
  std::unordered_multimap<uint64_t, hb_tmap_entry> tmap_cache;   // encoded TMA descriptors by argument hash
  // collectives
  void* nccl_comm = nullptr;
  int world = 1, rank = 0;
  hb_p2p_state p2p;
  // grow-only device buffers owned by the context
  void* scratch[HB_NUM_SCRATCH] = {};
  size_t scratch_bytes[HB_NUM_SCRATCH] = {};
  std::vector<void*> allocations;
  // RoPE angle table (cos, sin) for the last (seq, head_dim, base, pos0) used
  void* rope_table = nullptr;
  size_t rope_table_bytes = 0;
  int64_t rope_seq = 0, rope_head_dim = 0, rope_pos0 = 0;
  float rope_base = 0.f;
};

// Launch with the programmatic-stream-serialization attribute: the kernel may begin while the
// kernel in front of it on the stream is still running, and must execute `griddepcontrol.wait`
// before its first access to memory (the wait returns when that kernel has completed and its
// writes are visible).  What is gained is the launch latency between two dependent kernels, which
// dominates a step made of kernels of a few microseconds.
template <typename... KArgs, typename... Args>
inline cudaError_t hb_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                       Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

hb_status hb_fail(hb_ctx* ctx, hb_status code, const char* fmt, ...);
hb_status hb_check_cuda(hb_ctx* ctx, cudaError_t e, const char* what);
#define HB_CUDA(ctx, call)                                        \
  do {                                                            \
    cudaError_t e__ = (call);                                     \
    if (e__ != cudaSuccess) return hb_check_cuda(ctx, e__, #call); \
  } while (0)
// Drains every stream the context may have queued work on (before freeing its memory).
hb_status hb_quiesce(hb_ctx* ctx);
// Grow-only scratch buffer `slot` on the context's device.
hb_status hb_get_scratch(hb_ctx* ctx, int slot, size_t bytes, void** out);
// Copy streams and `n` ordering events for the pipelined host-buffer entry points.
hb_status hb_host_pipe(hb_ctx* ctx, int n, cudaEvent_t** events);

// cuTensorMapEncodeTiled fetched through the runtime (no link against libcuda).
// dims/strides innermost first; strides in bytes for dims 1..rank-1.
hb_status hb_make_tensor_map(hb_ctx* ctx, CUtensorMap* out, CUtensorMapDataType dt, int rank,
                             const void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                             const uint32_t* box, CUtensorMapSwizzle swizzle);

std::string hb_tune_key(const hb_op_desc& d, int sm_count, const std::string& gpu);
int hb_attention_cached_choice(hb_ctx* ctx, int64_t batch, int64_t seq, int64_t hq, int64_t hkv, int causal);

// Kernel launchers (each validates nothing: callers validated already).
struct hb_gemm_args {
  const void* A;
  const void* B;
  void* C;
  int64_t M, N, K;
  int64_t lda, ldb, ldc;   // elements
  int a_mn_major, b_mn_major;
  int epilogue;
  const void* residual;
  int64_t ldr;
  int b_is_weights;        // HB_MATMUL_WEIGHTS_B: nothing in flight writes B
  // rows of A published block by block while the kernel runs (see hb_matmul_gathered)
  const uint32_t* ready;
  uint32_t ready_epoch, ready_spin;
  int ready_rows, perm_world, perm_rank;
};
hb_status hb_launch_gemm_bf16(hb_ctx* ctx, const hb_gemm_args& a, int config_id);
hb_status hb_launch_gemm_f32(hb_ctx* ctx, const hb_gemm_args& a);
int hb_gemm_pick_config(hb_ctx* ctx, const hb_gemm_args& a);
// Split-K path for M <= 64 (decode-shaped) products.
bool hb_gemm_skinny_applicable(const hb_gemm_args& a);
hb_status hb_launch_gemm_skinny(hb_ctx* ctx, const hb_gemm_args& a);
// Same with the grid (persistent CTAs) and the k-blocks per ring stage given (the autotuner's axes).
hb_status hb_launch_gemm_skinny_cfg(hb_ctx* ctx, const hb_gemm_args& a, int grid_cap, int kps);
bool hb_skinny_cached_choice(hb_ctx* ctx, const hb_gemm_args& a, int* grid, int* kps);
// grid_cap <= 0: one CTA per SM; kps <= 0: the default (2).
void hb_gemm_skinny_plan(int sm_count, int64_t M, int64_t N, int64_t K, int grid_cap, int kps, int* grid, int* max_seg,
                         size_t* partial_floats, int* tiles);
hb_status hb_launch_gemm_skinny_raw(hb_ctx* ctx, cudaStream_t stream, const hb_gemm_args& a, float* partial, int* tickets,
                                    int grid, int max_seg, int tiles, int kps, int32_t* status);
