// Shared host-side helpers of the lightop_b200 C-ABI library.
#pragma once
#include <cuda_runtime.h>
#include <utility>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <atomic>
#include "../../include/lightop_b200.h"

namespace lo {

// Thread-local message returned by lo_last_error().
void set_error(const char *fmt, ...);

inline int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  set_error("%s", buf);
  return code;
}

#define LO_REQUIRE(cond, ...)                                             \
  do {                                                                    \
    if (!(cond)) return ::lo::fail(LO_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

#define LO_CUDA_OK(expr)                                                           \
  do {                                                                             \
    cudaError_t e__ = (expr);                                                      \
    if (e__ != cudaSuccess)                                                        \
      return ::lo::fail(LO_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

#define LO_LAUNCH_OK(what)                                                            \
  do {                                                                                \
    ::lo::g_launch_count.fetch_add(1, std::memory_order_relaxed);                     \
    cudaError_t e__ = cudaGetLastError();                                             \
    if (e__ != cudaSuccess)                                                           \
      return ::lo::fail(LO_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e__)); \
  } while (0)

// Kernels launched by this library since it was loaded (lo_launch_count): every launch site counts itself.
extern std::atomic<long long> g_launch_count;

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

int sm_count();

// ---------------------------------------------------------------------------
// Internal kernels shared between translation units
// ---------------------------------------------------------------------------

// One entry per unit of grouped-GEMM work along the token axis: up to 128
// expert-sorted rows of one expert.  expert < 0 marks a chunk whose output rows
// are to be zeroed.
struct Chunk {
  int32_t expert;
  int32_t row0;   // first position in sorted_ids
  int32_t rows;   // positions covered (<= the chunk size of the table); validity of each is the sentinel test
  int32_t pad;    // chunks of the same expert that follow (non-zero: the next chunk reads the same weight tiles, keep them in L2)
};

// Align + (optionally) chunk table, see routing.cu.
int launch_align(const void *topk_ids, int ids_dtype, int64_t numel, int num_experts, int block_size,
                 const int32_t *expert_map, int map_mode, int32_t *sorted_ids, int64_t sorted_capacity,
                 int32_t *expert_ids, int64_t expert_ids_capacity, int32_t *num_tokens_post_pad,
                 Chunk *chunks, int32_t *num_chunks, int64_t chunk_capacity, int32_t *inv_pos,
                 int chunk_max, cudaStream_t stream);

// Group quantisation of bf16 rows [M, H] written straight into the expert-sorted layout:
// the int8 row and its scales of token t go to every position inv_pos[t * topk + j] >= 0.  quant.cu
int launch_group_quant_scatter(const void *x, int64_t M, int64_t H, int topk, const int32_t *inv_pos, float eps,
                               int8_t *q_sorted, float *s_sorted, cudaStream_t stream);

// Per-token (whole-row) quantisation; with inv_pos the result goes to the token's sorted positions
// (q_out [positions, K], s_out [positions]), without it to row `token`.  quant.cu
int launch_token_quant(const void *x, int x_dtype, int64_t M, int64_t K, int topk, const int32_t *inv_pos, int8_t *q,
                       float *s, cudaStream_t stream);

// act = bf16(bf16(silu(gate)) * up) of bf16 rows [rows, 2*d], then per-token quantisation.  Rows at or
// beyond *num_rows_dev and rows whose row_ids entry is a padding sentinel are skipped (both optional).  quant.cu
// With group_counts the rows form [groups, group_rows] and only the first group_counts[g] rows of group g exist.
int launch_silu_mul_token_quant(const void *in, int64_t rows, int64_t d, const int32_t *row_ids, int64_t numel_valid,
                                const int32_t *num_rows_dev, int8_t *q, float *s, cudaStream_t stream,
                                int64_t group_rows = 0, const int32_t *group_counts = nullptr);

// Copy int8 rows and their scales into sorted-position order: row(pos) = sorted_ids[pos] / top_k.
// scales_per_row = 0 means K / 128 (block scales); 1 is the per-token format.  a_stride = 0 means K bytes between
// source rows; with a_scale == nullptr the scales of a row follow it inside its a_stride-byte record.  reduce.cu
int launch_permute_rows(const int8_t *A, const float *a_scale, int64_t rows_a, int64_t K, const int32_t *sorted_ids,
                        int64_t sorted_capacity, const int32_t *num_tokens_post_pad, int64_t numel_valid, int top_k,
                        int8_t *A_sorted, float *a_scale_sorted, cudaStream_t stream, int64_t scales_per_row = 0,
                        int64_t a_stride = 0);

// Expert id and routed weight of packed dispatch records (lo_ep_dispatch_pack) into contiguous arrays.  reduce.cu
int launch_ep_unpack_meta(const uint8_t *packed, int64_t rows, int64_t stride, int64_t meta_off, int32_t *row_expert,
                          float *row_weight, cudaStream_t stream, const int32_t *seg_first = nullptr,
                          const int64_t *seg_ret = nullptr, int world = 0, int64_t ret_row_bytes = 0,
                          int64_t *row_dst = nullptr);

// Chunk table from an existing (expert_ids, num_tokens_post_pad) pair, see routing.cu.
int launch_chunks_from_blocks(const int32_t *expert_ids, const int32_t *num_tokens_post_pad,
                              int block_size, int64_t max_blocks, Chunk *chunks, int32_t *num_chunks,
                              cudaStream_t stream);

// GEMM_GATE_UP / GEMM_SINGLE: 128x128 block scales (a_scale [rows, K/128], b_scale [E, N/128, K/128]).
// GEMM_CHANNEL: one scale per token and per output channel (a_scale [rows], b_scale [E, N]); bf16 output
// like GEMM_SINGLE.  In both bf16-output modes sorted_ids may be null: the id of a row is then its position.
enum GemmMode { GEMM_GATE_UP = 0, GEMM_SINGLE = 1, GEMM_CHANNEL = 2 };

struct GemmArgs {
  const int8_t *A;          // [rows_a, K] int8, rows in sorted-position order (row = position in sorted_ids)
  const float *a_scale;     // [rows_a, K/128]
  int64_t rows_a;
  int max_chunk_rows;       // upper bound of Chunk::rows (0 = 128); selects the shared-memory staging depth
  const int8_t *B;          // [E, n_rows_per_expert, K] int8
  const float *b_scale;     // [E, n_rows_per_expert/128, K/128]
  int E;
  int64_t n_rows_per_expert;   // 2I for gate_up, N for single
  int64_t n_store;             // 0 = n_rows_per_expert; output row length when N is not a multiple of 128 (E == 1 only)
  int64_t K;
  int n_tiles;              // 128-row output tiles per item: I/128 (gate_up) or N/128
  const int32_t *sorted_ids;
  int64_t numel_valid;      // sorted ids >= this are padding
  const Chunk *chunks;
  const int32_t *num_chunks;
  // outputs
  int8_t *act_q;            // gate_up: [positions, I]
  float *act_s;             // gate_up: [positions, I/128]
  __nv_bfloat16 *C;         // single: [numel_valid, N], row = sorted id
  const float *topk_weights;   // flat [numel_valid] or null
  int weight_mode;
  float act_eps;            // eps of the fused re-quantisation, already rounded to bf16
  int32_t *status;          // device word, set non-zero on a wait that ran out (may be null)
  int out_by_position;      // bf16 output row = sorted position (ids still select validity and the routed weight)
  // single (block-scaled) only: address of output row `sorted id`, one entry per id, instead of C + id * N.  The rows
  // may lie in another GPU's memory (a peer mapping): the epilogue writes them with plain 16-byte stores.
  const int64_t *row_dst;
};

int launch_grouped_gemm(GemmMode mode, const GemmArgs &args, cudaStream_t stream);

#ifdef __CUDACC__
// Programmatic dependent launch.  A kernel launched with launch_dependent() may start while the kernel before it
// in the stream is still running; it must call dependency_wait() before it touches anything that kernel writes
// (the call returns once the earlier grid has completed and its writes are visible; in a launch without the
// attribute it returns at once).  dependency_release() in the earlier kernel lets the next grid's blocks become
// resident as soon as every block of this grid has passed the call.
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Lanes of the warp that hold the same expert as this lane (lanes without an expert match one another).
// With many steps per warp the mask is built from one ballot per bit of the expert id: the match
// instruction proper has a throughput of the order of one warp per ~64 cycles and SM here, which made it the
// bottleneck at prefill sizes; with a few steps per warp (decode sizes) its single round trip is faster
// than the chain of ballots (nbits <= 0 selects it).
__device__ __forceinline__ unsigned peers_of(int e, int nbits) {
  if (nbits <= 0) return __match_any_sync(0xffffffffu, e);
  const unsigned has = __ballot_sync(0xffffffffu, e >= 0);
  unsigned peers = e >= 0 ? has : ~has;
  for (int b = 0; b < nbits; ++b) {
    const unsigned set = __ballot_sync(0xffffffffu, (e >> b) & 1);
    peers &= ((e >> b) & 1) ? set : ~set;
  }
  return peers;
}
#endif

// Top-k sum of the fused layers.  A slot is skipped under the alignment kernel's rule: its id lies outside
// [0, num_experts) or (with an expert_map) maps outside [0, num_local); such rows were never written.  reduce.cu
int launch_moe_sum_masked(const __nv_bfloat16 *in, __nv_bfloat16 *out, const __nv_bfloat16 *bias,
                          int64_t M, int topk, int64_t H, float factor, const void *topk_ids,
                          int ids_dtype, const int32_t *expert_map, int num_experts, int num_local, cudaStream_t stream);

}  // namespace lo
