// Host-side composition of the fused block-INT8 MoE layer and of the stand-alone
// grouped GEMM entry point.  Everything here only carves the caller's workspace
// and enqueues kernels on the caller's stream.
#include "common.h"
#include <mutex>

namespace lo {
float round_eps_to_dtype(float eps, int dtype);   // quant.cu
namespace {

constexpr int64_t ALIGN_BYTES = 256;
constexpr int FUSED_ALIGN_BLOCK = 16;   // expert segments start on multiples of the MMA N granule

struct Carver {
  uint8_t *base;
  size_t off = 0;
  explicit Carver(void *b) : base(static_cast<uint8_t *>(b)) {}
  template <typename T> T *take(int64_t count) {
    T *p = base ? reinterpret_cast<T *>(base + off) : nullptr;
    off += (size_t)round_up(count * (int64_t)sizeof(T), ALIGN_BYTES);
    return p;
  }
};

struct FusedLayout {
  int8_t *xq;           // [sorted_cap, H] quantised activations in sorted-position order
  float *xs;            // [sorted_cap, H/128]
  int32_t *header;      // [0] num_tokens_post_pad, [1] num_chunks
  int32_t *sorted_ids;
  int32_t *inv_pos;     // [M*topk] position of every (token, slot), -1 if dropped
  Chunk *chunks;
  int8_t *act_q;
  float *act_s;
  int64_t sorted_cap;
  int64_t chunk_cap;
  size_t bytes;
};

FusedLayout carve_fused(void *ws, int64_t M, int num_experts_for_align, int topk, int64_t H, int64_t I) {
  FusedLayout L;
  Carver c(ws);
  const int64_t numel = M * topk;
  L.sorted_cap = numel + (int64_t)num_experts_for_align * (FUSED_ALIGN_BLOCK - 1);
  L.chunk_cap = numel / 32 + num_experts_for_align + 1;   // enough for the smallest chunk size (32 rows)
  L.header = c.take<int32_t>(64);
  L.xq = c.take<int8_t>(L.sorted_cap * H);
  L.xs = c.take<float>(L.sorted_cap * (H / 128));
  L.sorted_ids = c.take<int32_t>(L.sorted_cap);
  L.inv_pos = c.take<int32_t>(numel);
  L.chunks = c.take<Chunk>(L.chunk_cap);
  L.act_q = c.take<int8_t>(L.sorted_cap * I);
  L.act_s = c.take<float>(L.sorted_cap * (I / 128));
  L.bytes = c.off;
  return L;
}

// Chunk sizes of the block-scaled layer, by the rows an expert gets on average (rows / experts), measured at the
// DeepSeek-V3 shape.  The GEMM is instantiated per chunk cap and the caps differ in what fits beside the operands:
// chunks of <= 64 rows leave room for 12 weight slots and 8 partial buffers, <= 128 rows for 7 and 4, <= 160 rows for 5
// and 3.
//   <= 48 rows per expert : 64-row chunks.  A weight-streaming call wants the deep rings, and the few experts that do
//                           get more rows simply have a second chunk (-8 % from 96 to 512 tokens, -4 % at 1536).
//   49 .. 119             : 128-row chunks (-9 % at 64 rows per expert, -2 % at 112 against the 160-row table).
//   >= 120                : 160-row chunks, the widest whose partial buffers still number three: at 128 rows per expert
//                           half of the experts have a few rows more than 128, and a second chunk means a second pass
//                           over the expert's weights (-17 % at 128 rows per expert against the 128-row table).
constexpr int CHUNK_ROWS = 128;
constexpr int CHUNK_ROWS_WIDE = 160;
constexpr int CHUNK_ROWS_SMALL = 64;
inline int chunk_rows_for(int64_t rows, int experts) {
  const int64_t avg = rows / experts;
  return avg >= 120 ? CHUNK_ROWS_WIDE : (avg <= 48 ? CHUNK_ROWS_SMALL : CHUNK_ROWS);
}

// Optional per-stage timing of the fused call (cudaEvents recorded between its five kernels).
struct StageProfile {
  bool enabled = false;
  bool created = false;
  bool recorded = false;
  cudaEvent_t ev[6];
};
thread_local StageProfile g_prof;

inline void prof_mark(int i, cudaStream_t st) {
  if (g_prof.enabled && g_prof.created) cudaEventRecord(g_prof.ev[i], st);
}

}  // namespace
}  // namespace lo

extern "C" int lo_profile_enable(int on) {
  using namespace lo;
  if (on && !g_prof.created) {
    for (int i = 0; i < 6; ++i) LO_CUDA_OK(cudaEventCreate(&g_prof.ev[i]));
    g_prof.created = true;
  }
  g_prof.enabled = on != 0;
  g_prof.recorded = false;
  return LO_OK;
}

extern "C" int lo_profile_read(float *ms5) {
  using namespace lo;
  LO_REQUIRE(ms5 != nullptr, "profile read: null output");
  LO_REQUIRE(g_prof.created && g_prof.recorded, "profile read: no fused call was recorded on this thread");
  LO_CUDA_OK(cudaEventSynchronize(g_prof.ev[5]));
  for (int i = 0; i < 5; ++i) LO_CUDA_OK(cudaEventElapsedTime(&ms5[i], g_prof.ev[i], g_prof.ev[i + 1]));
  return LO_OK;
}

extern "C" size_t lo_fused_moe_workspace_bytes(int64_t M, int E_local, int global_num_experts, int topk, int64_t H,
                                               int64_t I) {
  const int e = global_num_experts > E_local ? global_num_experts : E_local;
  return lo::carve_fused(nullptr, M, e, topk, H, I).bytes;
}

extern "C" int lo_fused_moe_workspace_layout(int64_t M, int E_local, int global_num_experts, int topk, int64_t H,
                                            int64_t I, int64_t *out8) {
  using namespace lo;
  LO_REQUIRE(out8 != nullptr, "workspace layout: null output");
  const int e = global_num_experts > E_local ? global_num_experts : E_local;
  uint8_t *base = reinterpret_cast<uint8_t *>(uintptr_t(4096));   // any non-null base: only differences are used
  FusedLayout L = carve_fused(base, M, e, topk, H, I);
  out8[0] = reinterpret_cast<uint8_t *>(L.header) - base;
  out8[1] = reinterpret_cast<uint8_t *>(L.xq) - base;
  out8[2] = reinterpret_cast<uint8_t *>(L.xs) - base;
  out8[3] = reinterpret_cast<uint8_t *>(L.sorted_ids) - base;
  out8[4] = reinterpret_cast<uint8_t *>(L.chunks) - base;
  out8[5] = reinterpret_cast<uint8_t *>(L.act_q) - base;
  out8[6] = reinterpret_cast<uint8_t *>(L.act_s) - base;
  out8[7] = L.sorted_cap;
  return LO_OK;
}

extern "C" int lo_fused_moe_block_int8(const void *x, const int8_t *w1, const int8_t *w2, const float *w1_scale,
                                       const float *w2_scale, const float *topk_weights, const void *topk_ids,
                                       int ids_dtype, const int32_t *expert_map, int global_num_experts, int64_t M,
                                       int E_local, int topk, int64_t H, int64_t I, void *cache3,
                                       const void *shared_output, void *out, int apply_router_weight_on_input,
                                       float routed_scaling_factor, void *workspace, size_t workspace_bytes,
                                       int32_t *status, void *stream) {
  using namespace lo;
  LO_REQUIRE(M >= 0 && E_local >= 1 && topk >= 1, "fused moe: bad shape");
  if (M == 0) return LO_OK;
  LO_REQUIRE(x && w1 && w2 && w1_scale && w2_scale && topk_weights && topk_ids && cache3 && out && workspace,
             "fused moe: null pointer");
  LO_REQUIRE(H % 128 == 0 && I % 128 == 0, "fused moe: hidden (%lld) and intermediate (%lld) sizes must be multiples of 128",
             (long long)H, (long long)I);
  LO_REQUIRE(ids_dtype == LO_I32 || ids_dtype == LO_I64, "fused moe: topk_ids must be int32 or int64");
  LO_REQUIRE(!apply_router_weight_on_input || topk == 1, "fused moe: apply_router_weight_on_input requires topk == 1");
  LO_REQUIRE(M * topk < (1LL << 30), "fused moe: too many (token, slot) pairs; split the call into chunks");
  if (global_num_experts <= 0) global_num_experts = E_local;
  LO_REQUIRE(expert_map != nullptr || global_num_experts == E_local, "fused moe: global_num_experts != E needs an expert_map");
  const int align_E = expert_map ? global_num_experts : E_local;
  LO_REQUIRE(align_E <= 1024, "fused moe: more than 1024 experts");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & (ALIGN_BYTES - 1)) == 0, "fused moe: workspace must be 256-byte aligned");
  FusedLayout L = carve_fused(workspace, M, align_E, topk, H, I);
  LO_REQUIRE(workspace_bytes >= L.bytes, "fused moe: workspace of %zu bytes, %zu needed", workspace_bytes, L.bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t numel = M * topk;
  int rc;

  const int chunk_max = chunk_rows_for(numel, align_E);
  // 1. expert-major stable order, chunk table, position of every (token, slot)
  prof_mark(0, st);
  rc = launch_align(topk_ids, ids_dtype, numel, align_E, FUSED_ALIGN_BLOCK, expert_map, expert_map ? 1 : 0,
                    L.sorted_ids, L.sorted_cap, nullptr, 0, L.header, L.chunks, L.header + 1, L.chunk_cap, L.inv_pos,
                    chunk_max, st);
  if (rc != LO_OK) return rc;

  // 2. activations -> int8 + per-128 scales, written once per routed slot into sorted order so
  //    that every chunk of the grouped GEMM is a run of consecutive rows (one TMA box)
  prof_mark(1, st);
  rc = launch_group_quant_scatter(x, M, H, topk, L.inv_pos, 1e-10f, L.xq, L.xs, st);
  if (rc != LO_OK) return rc;

  // 3. gate_up GEMM, SiLU*mul and re-quantisation in the epilogue -> act_q/act_s in sorted order
  prof_mark(2, st);
  GemmArgs g1{};
  g1.A = L.xq; g1.a_scale = L.xs; g1.rows_a = L.sorted_cap;
  g1.max_chunk_rows = (int)(M < chunk_max ? M : chunk_max);   // an expert receives at most one row per token
  g1.B = w1; g1.b_scale = w1_scale; g1.E = E_local;
  g1.n_rows_per_expert = 2 * I; g1.K = H; g1.n_tiles = (int)(I / 128);
  g1.sorted_ids = L.sorted_ids; g1.numel_valid = numel;
  g1.chunks = L.chunks; g1.num_chunks = L.header + 1;
  g1.act_q = L.act_q; g1.act_s = L.act_s; g1.C = nullptr;
  g1.topk_weights = topk_weights;
  g1.weight_mode = apply_router_weight_on_input ? LO_WEIGHT_FP32 : LO_WEIGHT_NONE;
  g1.act_eps = round_eps_to_dtype(1e-10f, LO_BF16);
  g1.status = status;
  rc = launch_grouped_gemm(GEMM_GATE_UP, g1, st);
  if (rc != LO_OK) return rc;

  // 4. down GEMM, routed weight in the epilogue -> cache3[token, slot, :]
  prof_mark(3, st);
  GemmArgs g2{};
  g2.A = L.act_q; g2.a_scale = L.act_s; g2.rows_a = L.sorted_cap;
  g2.max_chunk_rows = g1.max_chunk_rows; g2.B = w2; g2.b_scale = w2_scale; g2.E = E_local;
  g2.n_rows_per_expert = H; g2.K = I; g2.n_tiles = (int)(H / 128);
  g2.sorted_ids = L.sorted_ids; g2.numel_valid = numel;
  g2.chunks = L.chunks; g2.num_chunks = L.header + 1;
  g2.C = static_cast<__nv_bfloat16 *>(cache3);
  g2.topk_weights = topk_weights;
  g2.weight_mode = apply_router_weight_on_input ? LO_WEIGHT_NONE : LO_WEIGHT_BF16_PRODUCT;
  g2.act_eps = 0.f;
  g2.status = status;
  rc = launch_grouped_gemm(GEMM_SINGLE, g2, st);
  if (rc != LO_OK) return rc;

  // 5. top-k reduction (slots of non-local experts are skipped, their rows were never written)
  prof_mark(4, st);
  rc = launch_moe_sum_masked(static_cast<const __nv_bfloat16 *>(cache3), static_cast<__nv_bfloat16 *>(out),
                             static_cast<const __nv_bfloat16 *>(shared_output), M, topk, H, routed_scaling_factor,
                             topk_ids, ids_dtype, expert_map, align_E, E_local, st);
  prof_mark(5, st);
  if (g_prof.enabled && g_prof.created) g_prof.recorded = true;
  return rc;
}

namespace lo {
namespace {
struct GemmWs {
  int32_t *num_chunks;
  Chunk *chunks;
  int8_t *a_sorted;
  float *as_sorted;
  size_t bytes;
};
GemmWs carve_gemm(void *ws, int64_t sorted_capacity, int block_size, int64_t K) {
  GemmWs W;
  Carver c(ws);
  const int64_t blocks = ceil_div(sorted_capacity, block_size);
  const int per_block = block_size <= 128 ? 1 : block_size / 128;
  W.num_chunks = c.take<int32_t>(64);
  W.chunks = c.take<Chunk>(blocks * per_block + 1);
  W.a_sorted = c.take<int8_t>(sorted_capacity * K);
  W.as_sorted = c.take<float>(sorted_capacity * (K / 128));
  W.bytes = c.off;
  return W;
}
}  // namespace
}  // namespace lo

extern "C" size_t lo_grouped_gemm_workspace_bytes(int64_t sorted_capacity, int block_size, int64_t K) {
  if (block_size <= 0 || sorted_capacity <= 0 || K <= 0) return 0;
  return lo::carve_gemm(nullptr, sorted_capacity, block_size, K).bytes;
}

namespace lo {
namespace {
// Both scale formats of the stand-alone grouped GEMM: chunk table from the caller's block table, rows and
// scales permuted into sorted order, then the kernel of the format.
int grouped_gemm_on_blocks(GemmMode mode, const int8_t *A, const float *a_scale, int64_t rows_a, const int8_t *B,
                           const float *b_scale, int E, int64_t N, int64_t K, void *C, const float *topk_weights,
                           int weight_mode, const int32_t *sorted_ids, int64_t sorted_capacity,
                           const int32_t *expert_ids, const int32_t *num_tokens_post_pad, int64_t numel_valid,
                           int top_k, int block_size, void *workspace, size_t workspace_bytes, void *stream) {
  LO_REQUIRE(A && a_scale && B && b_scale && C && sorted_ids && expert_ids && num_tokens_post_pad && workspace,
             "grouped gemm: null pointer");
  LO_REQUIRE(block_size >= 1 && (block_size <= 128 || block_size % 128 == 0),
             "grouped gemm: block_size %d must be <= 128 or a multiple of 128", block_size);
  LO_REQUIRE(top_k >= 1 && E >= 1 && rows_a >= 0 && sorted_capacity >= 1, "grouped gemm: bad shape");
  LO_REQUIRE(K % 128 == 0 && N % 128 == 0, "grouped gemm: N and K must be multiples of 128");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & (ALIGN_BYTES - 1)) == 0, "grouped gemm: workspace must be 256-byte aligned");
  GemmWs W = carve_gemm(workspace, sorted_capacity, block_size, K);   // sized for block scales; per-token scales need less
  LO_REQUIRE(workspace_bytes >= W.bytes, "grouped gemm: workspace of %zu bytes, %zu needed", workspace_bytes, W.bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t max_blocks = ceil_div(sorted_capacity, block_size);
  int rc = launch_chunks_from_blocks(expert_ids, num_tokens_post_pad, block_size, max_blocks, W.chunks, W.num_chunks, st);
  if (rc != LO_OK) return rc;
  rc = launch_permute_rows(A, a_scale, rows_a, K, sorted_ids, sorted_capacity, num_tokens_post_pad, numel_valid, top_k,
                           W.a_sorted, W.as_sorted, st, mode == GEMM_CHANNEL ? 1 : 0);
  if (rc != LO_OK) return rc;
  GemmArgs g{};
  g.A = W.a_sorted; g.a_scale = W.as_sorted; g.rows_a = sorted_capacity;
  g.max_chunk_rows = block_size < 128 ? block_size : 128; g.B = B; g.b_scale = b_scale; g.E = E;
  g.n_rows_per_expert = N; g.K = K; g.n_tiles = (int)(N / 128);
  g.sorted_ids = sorted_ids; g.numel_valid = numel_valid;
  g.chunks = W.chunks; g.num_chunks = W.num_chunks;
  g.C = static_cast<__nv_bfloat16 *>(C);
  g.topk_weights = topk_weights; g.weight_mode = weight_mode; g.act_eps = 0.f; g.status = nullptr;
  return launch_grouped_gemm(mode, g, st);
}
}  // namespace
}  // namespace lo

extern "C" int lo_moe_grouped_gemm_i8_block(const int8_t *A, const float *a_scale, int64_t rows_a, const int8_t *B,
                                            const float *b_scale, int E, int64_t N, int64_t K, void *C,
                                            const float *topk_weights, int weight_mode, const int32_t *sorted_ids,
                                            int64_t sorted_capacity, const int32_t *expert_ids,
                                            const int32_t *num_tokens_post_pad, int64_t numel_valid, int top_k,
                                            int block_size, void *workspace, size_t workspace_bytes, void *stream) {
  return lo::grouped_gemm_on_blocks(lo::GEMM_SINGLE, A, a_scale, rows_a, B, b_scale, E, N, K, C, topk_weights, weight_mode,
                                    sorted_ids, sorted_capacity, expert_ids, num_tokens_post_pad, numel_valid, top_k,
                                    block_size, workspace, workspace_bytes, stream);
}

// Per-channel form of the grouped GEMM: a_scale [rows_a] (one per token), b_scale [E, N].
extern "C" int lo_moe_grouped_gemm_i8_channel(const int8_t *A, const float *a_scale, int64_t rows_a, const int8_t *B,
                                              const float *b_scale, int E, int64_t N, int64_t K, void *C,
                                              const float *topk_weights, int weight_mode, const int32_t *sorted_ids,
                                              int64_t sorted_capacity, const int32_t *expert_ids,
                                              const int32_t *num_tokens_post_pad, int64_t numel_valid, int top_k,
                                              int block_size, void *workspace, size_t workspace_bytes, void *stream) {
  return lo::grouped_gemm_on_blocks(lo::GEMM_CHANNEL, A, a_scale, rows_a, B, b_scale, E, N, K, C, topk_weights, weight_mode,
                                    sorted_ids, sorted_capacity, expert_ids, num_tokens_post_pad, numel_valid, top_k,
                                    block_size, workspace, workspace_bytes, stream);
}

// ---------------------------------------------------------------------------
// Fused layer without any caller-supplied or allocated scratch.
//
// Some hosts of this library have no way to obtain device memory at the moment they need the
// layer: a serving thread that must not trigger the implicit device-wide synchronisation of
// cudaMalloc, a plugin that is handed raw pointers by a runtime which owns the only allocator,
// a foreign-language binding (cgo / JNI / Rust FFI) that was given no allocator handle.  For
// them the scratch of the fused layer lives in a fixed array that is part of the library image:
// every GPU that loads the library reserves LO_NOALLOC_SCRATCH_BYTES for it until the process ends.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_noalloc_scratch[LO_NOALLOC_SCRATCH_BYTES];

namespace lo {
namespace {
constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
void *g_noalloc_ptr[kMaxDevices] = {};   // device address of g_noalloc_scratch, per device ordinal

// The name g_noalloc_scratch is a host-side handle here, not an address a kernel may use: the
// device address is looked up once per device, with that device current.
int noalloc_scratch(void **out) {
  int dev = -1;
  LO_CUDA_OK(cudaGetDevice(&dev));
  LO_REQUIRE(dev >= 0 && dev < kMaxDevices, "no-alloc fused moe: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void *ptr = nullptr;
    LO_CUDA_OK(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    LO_REQUIRE(ptr != nullptr, "no-alloc fused moe: the scratch symbol has no device address");
    g_noalloc_ptr[dev] = ptr;
  }
  *out = g_noalloc_ptr[dev];
  return LO_OK;
}
}  // namespace
}  // namespace lo

extern "C" int lo_fused_moe_block_int8_noalloc(const void *x, const int8_t *w1, const int8_t *w2,
                                               const float *w1_scale, const float *w2_scale,
                                               const float *topk_weights, const void *topk_ids, int ids_dtype,
                                               const int32_t *expert_map, int global_num_experts, int64_t M,
                                               int E_local, int topk, int64_t H, int64_t I, void *cache3,
                                               const void *shared_output, void *out,
                                               int apply_router_weight_on_input, float routed_scaling_factor,
                                               int32_t *status, void *stream) {
  using namespace lo;
  LO_REQUIRE(M >= 0 && E_local >= 1 && topk >= 1 && H >= 128 && I >= 128, "no-alloc fused moe: bad shape");
  const size_t need = lo_fused_moe_workspace_bytes(M, E_local, global_num_experts, topk, H, I);
  if (need > (size_t)LO_NOALLOC_SCRATCH_BYTES)
    return fail(LO_ERR_INVALID_ARGUMENT,
                "no-alloc fused moe: this shape needs %zu bytes of scratch, the built-in array holds %zu; "
                "use fewer tokens per call or lo_fused_moe_block_int8 with a caller-owned workspace",
                need, (size_t)LO_NOALLOC_SCRATCH_BYTES);
  void *scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != LO_OK) return rc;
  // Nothing in the scratch has to start at zero: every region a kernel reads for a result was written
  // earlier in the same call (sentinel fill, header, chunk table, sorted rows), so the previous call's
  // contents that remain in it are never interpreted.
  return lo_fused_moe_block_int8(x, w1, w2, w1_scale, w2_scale, topk_weights, topk_ids, ids_dtype, expert_map,
                                 global_num_experts, M, E_local, topk, H, I, cache3, shared_output, out,
                                 apply_router_weight_on_input, routed_scaling_factor, scratch, need, status, stream);
}

// ---------------------------------------------------------------------------
// Per-channel W8A8 mode of the same layer: one scale per token (activations) and one per output
// channel (weights).  The GEMMs accumulate int32 over the whole K extent on the tensor core and
// apply both scales once in the epilogue; SiLU*mul and the per-token re-quantisation need the
// maximum of a whole row, so they run as a kernel of their own between the two GEMMs, as in the
// reference (python/lightop/_lmslim_native/layers/fused_moe/int8.py:771-905).
// ---------------------------------------------------------------------------
namespace lo {
namespace {
struct ChannelLayout {
  int32_t *header;      // [0] num_tokens_post_pad, [1] num_chunks
  int8_t *xq;           // [sorted_cap, H]
  float *xs;            // [sorted_cap]
  int32_t *sorted_ids;
  int32_t *inv_pos;
  Chunk *chunks;
  __nv_bfloat16 *cache1;   // [sorted_cap, 2I] gate_up output by sorted position
  int8_t *act_q;        // [sorted_cap, I]
  float *act_s;         // [sorted_cap]
  int64_t sorted_cap;
  int64_t chunk_cap;
  size_t bytes;
};
ChannelLayout carve_channel(void *ws, int64_t M, int num_experts_for_align, int topk, int64_t H, int64_t I) {
  ChannelLayout L;
  Carver c(ws);
  const int64_t numel = M * topk;
  L.sorted_cap = numel + (int64_t)num_experts_for_align * (FUSED_ALIGN_BLOCK - 1);
  L.chunk_cap = numel / 32 + num_experts_for_align + 1;
  L.header = c.take<int32_t>(64);
  L.xq = c.take<int8_t>(L.sorted_cap * H);
  L.xs = c.take<float>(L.sorted_cap);
  L.sorted_ids = c.take<int32_t>(L.sorted_cap);
  L.inv_pos = c.take<int32_t>(numel);
  L.chunks = c.take<Chunk>(L.chunk_cap);
  L.cache1 = c.take<__nv_bfloat16>(L.sorted_cap * 2 * I);
  L.act_q = c.take<int8_t>(L.sorted_cap * I);
  L.act_s = c.take<float>(L.sorted_cap);
  L.bytes = c.off;
  return L;
}
}  // namespace
}  // namespace lo

extern "C" size_t lo_fused_moe_channel_workspace_bytes(int64_t M, int E_local, int global_num_experts, int topk,
                                                       int64_t H, int64_t I) {
  const int e = global_num_experts > E_local ? global_num_experts : E_local;
  return lo::carve_channel(nullptr, M, e, topk, H, I).bytes;
}

extern "C" int lo_fused_moe_channel_int8(const void *x, int x_dtype, const int8_t *w1, const int8_t *w2,
                                         const float *w1_scale, const float *w2_scale, const float *topk_weights,
                                         const void *topk_ids, int ids_dtype, const int32_t *expert_map,
                                         int global_num_experts, int64_t M, int E_local, int topk, int64_t H, int64_t I,
                                         void *cache3, const void *shared_output, void *out,
                                         int apply_router_weight_on_input, float routed_scaling_factor, void *workspace,
                                         size_t workspace_bytes, int32_t *status, void *stream) {
  using namespace lo;
  LO_REQUIRE(M >= 0 && E_local >= 1 && topk >= 1, "channel moe: bad shape");
  if (M == 0) return LO_OK;
  LO_REQUIRE(x && w1 && w2 && w1_scale && w2_scale && topk_weights && topk_ids && cache3 && out && workspace,
             "channel moe: null pointer");
  LO_REQUIRE(x_dtype == LO_BF16, "channel moe: activations must be bfloat16");
  LO_REQUIRE(H % 128 == 0 && I % 128 == 0, "channel moe: hidden (%lld) and intermediate (%lld) sizes must be multiples of 128",
             (long long)H, (long long)I);
  LO_REQUIRE(ids_dtype == LO_I32 || ids_dtype == LO_I64, "channel moe: topk_ids must be int32 or int64");
  LO_REQUIRE(!apply_router_weight_on_input || topk == 1, "channel moe: apply_router_weight_on_input requires topk == 1");
  LO_REQUIRE(M * topk < (1LL << 30), "channel moe: too many (token, slot) pairs; split the call into chunks");
  if (global_num_experts <= 0) global_num_experts = E_local;
  LO_REQUIRE(expert_map != nullptr || global_num_experts == E_local, "channel moe: global_num_experts != E needs an expert_map");
  const int align_E = expert_map ? global_num_experts : E_local;
  LO_REQUIRE(align_E <= 1024, "channel moe: more than 1024 experts");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & (ALIGN_BYTES - 1)) == 0, "channel moe: workspace must be 256-byte aligned");
  ChannelLayout L = carve_channel(workspace, M, align_E, topk, H, I);
  LO_REQUIRE(workspace_bytes >= L.bytes, "channel moe: workspace of %zu bytes, %zu needed", workspace_bytes, L.bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t numel = M * topk;
  // Largest chunk of one expert's rows handed to a CTA.  A chunk of up to 256 rows is one MMA N extent, so an
  // expert with 129..256 rows streams its weights once instead of once per 128-row chunk (the second pass
  // was found to miss L2 often), and an N = 256 MMA costs about 1.3x an N = 128 one.  The 256-row kernel
  // stages fewer K blocks ahead, so it is used only when experts are expected to receive that many rows.
  const int chunk_max = numel / align_E >= 64 ? 256 : 128;
  // 1. expert-major stable order, chunk table, position of every (token, slot)
  prof_mark(0, st);
  int rc = launch_align(topk_ids, ids_dtype, numel, align_E, FUSED_ALIGN_BLOCK, expert_map, expert_map ? 1 : 0,
                        L.sorted_ids, L.sorted_cap, nullptr, 0, L.header, L.chunks, L.header + 1, L.chunk_cap,
                        L.inv_pos, chunk_max, st);
  if (rc != LO_OK) return rc;
  // 2. per-token quantisation, written once per routed slot into sorted order
  prof_mark(1, st);
  rc = launch_token_quant(x, x_dtype, M, H, topk, L.inv_pos, L.xq, L.xs, st);
  if (rc != LO_OK) return rc;
  // 3. gate_up GEMM -> bf16 [position, 2I]
  prof_mark(2, st);
  GemmArgs g1{};
  g1.A = L.xq; g1.a_scale = L.xs; g1.rows_a = L.sorted_cap;
  g1.max_chunk_rows = (int)(M < chunk_max ? M : chunk_max);
  g1.B = w1; g1.b_scale = w1_scale; g1.E = E_local;
  g1.n_rows_per_expert = 2 * I; g1.K = H; g1.n_tiles = (int)(2 * I / 128);
  g1.sorted_ids = L.sorted_ids; g1.numel_valid = numel; g1.out_by_position = 1;
  g1.chunks = L.chunks; g1.num_chunks = L.header + 1;
  g1.C = L.cache1;
  g1.topk_weights = topk_weights;
  g1.weight_mode = apply_router_weight_on_input ? LO_WEIGHT_FP32 : LO_WEIGHT_NONE;
  g1.status = status;
  rc = launch_grouped_gemm(GEMM_CHANNEL, g1, st);
  if (rc != LO_OK) return rc;
  // SiLU*mul + per-token re-quantisation of the rows that exist (padding positions are skipped)
  rc = launch_silu_mul_token_quant(L.cache1, L.sorted_cap, I, L.sorted_ids, numel, L.header, L.act_q, L.act_s, st);
  if (rc != LO_OK) return rc;
  // 4. down GEMM, routed weight in the epilogue -> cache3[token, slot, :]
  prof_mark(3, st);
  GemmArgs g2{};
  g2.A = L.act_q; g2.a_scale = L.act_s; g2.rows_a = L.sorted_cap; g2.max_chunk_rows = g1.max_chunk_rows;
  g2.B = w2; g2.b_scale = w2_scale; g2.E = E_local;
  g2.n_rows_per_expert = H; g2.K = I; g2.n_tiles = (int)(H / 128);
  g2.sorted_ids = L.sorted_ids; g2.numel_valid = numel;
  g2.chunks = L.chunks; g2.num_chunks = L.header + 1;
  g2.C = static_cast<__nv_bfloat16 *>(cache3);
  g2.topk_weights = topk_weights;
  g2.weight_mode = apply_router_weight_on_input ? LO_WEIGHT_NONE : LO_WEIGHT_FP32;
  g2.status = status;
  rc = launch_grouped_gemm(GEMM_CHANNEL, g2, st);
  if (rc != LO_OK) return rc;
  // 5. top-k reduction
  prof_mark(4, st);
  rc = launch_moe_sum_masked(static_cast<const __nv_bfloat16 *>(cache3), static_cast<__nv_bfloat16 *>(out),
                             static_cast<const __nv_bfloat16 *>(shared_output), M, topk, H, routed_scaling_factor,
                             topk_ids, ids_dtype, expert_map, align_E, E_local, st);
  prof_mark(5, st);
  if (g_prof.enabled && g_prof.created) g_prof.recorded = true;
  return rc;
}

// ---------------------------------------------------------------------------
// Expert side of expert parallelism: rows arrive already quantised (int8 + group scales), each with
// the local expert that has to process it and, optionally, its routed weight.
// ---------------------------------------------------------------------------
namespace lo {
namespace {
// xs == nullptr: the rows are records of `x_stride` bytes, int8 row first, its group scales right behind it
int expert_rows_impl(const int8_t *xq, const float *xs, int64_t x_stride, const int32_t *row_expert,
                     const float *row_weight, const int8_t *w1, const int8_t *w2, const float *w1_scale,
                     const float *w2_scale, int64_t T, int E_local, int64_t H, int64_t I, void *out, void *workspace,
                     size_t workspace_bytes, int32_t *status, void *stream, const int64_t *row_dst = nullptr) {
  LO_REQUIRE(T >= 0 && E_local >= 1 && E_local <= 1024, "expert rows: bad shape");
  if (T == 0) return LO_OK;
  LO_REQUIRE(xq && row_expert && w1 && w2 && w1_scale && w2_scale && (out || row_dst) && workspace, "expert rows: null pointer");
  LO_REQUIRE(H % 128 == 0 && I % 128 == 0, "expert rows: hidden and intermediate sizes must be multiples of 128");
  LO_REQUIRE(T < (1LL << 30), "expert rows: too many rows");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & (ALIGN_BYTES - 1)) == 0, "expert rows: workspace must be 256-byte aligned");
  FusedLayout L = carve_fused(workspace, T, E_local, 1, H, I);
  LO_REQUIRE(workspace_bytes >= L.bytes, "expert rows: workspace of %zu bytes, %zu needed", workspace_bytes, L.bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // chunk sizes: the rule of lo_fused_moe_block_int8
  const int chunk_max = chunk_rows_for(T, E_local);
  // 1. expert-major stable order of the rows (ids outside [0, E_local) are dropped)
  int rc = launch_align(row_expert, LO_I32, T, E_local, FUSED_ALIGN_BLOCK, nullptr, 0, L.sorted_ids, L.sorted_cap,
                        nullptr, 0, L.header, L.chunks, L.header + 1, L.chunk_cap, nullptr, chunk_max, st);
  if (rc != LO_OK) return rc;
  // 2. rows and scales into sorted order
  rc = launch_permute_rows(xq, xs, T, H, L.sorted_ids, L.sorted_cap, L.header, T, 1, L.xq, L.xs, st, 0, x_stride);
  if (rc != LO_OK) return rc;
  GemmArgs g1{};
  g1.A = L.xq; g1.a_scale = L.xs; g1.rows_a = L.sorted_cap; g1.max_chunk_rows = (int)(T < chunk_max ? T : chunk_max);
  g1.B = w1; g1.b_scale = w1_scale; g1.E = E_local;
  g1.n_rows_per_expert = 2 * I; g1.K = H; g1.n_tiles = (int)(I / 128);
  g1.sorted_ids = L.sorted_ids; g1.numel_valid = T;
  g1.chunks = L.chunks; g1.num_chunks = L.header + 1;
  g1.act_q = L.act_q; g1.act_s = L.act_s;
  g1.weight_mode = LO_WEIGHT_NONE;
  g1.act_eps = round_eps_to_dtype(1e-10f, LO_BF16);
  g1.status = status;
  rc = launch_grouped_gemm(GEMM_GATE_UP, g1, st);
  if (rc != LO_OK) return rc;
  GemmArgs g2{};
  g2.A = L.act_q; g2.a_scale = L.act_s; g2.rows_a = L.sorted_cap; g2.max_chunk_rows = g1.max_chunk_rows;
  g2.B = w2; g2.b_scale = w2_scale; g2.E = E_local;
  g2.n_rows_per_expert = H; g2.K = I; g2.n_tiles = (int)(H / 128);
  g2.sorted_ids = L.sorted_ids; g2.numel_valid = T;
  g2.chunks = L.chunks; g2.num_chunks = L.header + 1;
  g2.C = static_cast<__nv_bfloat16 *>(out);      // top_k = 1: the sorted id is the row itself
  g2.row_dst = row_dst;                          // or: every row has an address of its own
  g2.topk_weights = row_weight;
  g2.weight_mode = row_weight ? LO_WEIGHT_BF16_PRODUCT : LO_WEIGHT_NONE;
  g2.status = status;
  return launch_grouped_gemm(GEMM_SINGLE, g2, st);
}
}  // namespace
}  // namespace lo

extern "C" int lo_expert_rows_block_int8(const int8_t *xq, const float *xs, const int32_t *row_expert,
                                         const float *row_weight, const int8_t *w1, const int8_t *w2,
                                         const float *w1_scale, const float *w2_scale, int64_t T, int E_local,
                                         int64_t H, int64_t I, void *out, void *workspace, size_t workspace_bytes,
                                         int32_t *status, void *stream) {
  LO_REQUIRE(xs != nullptr || T == 0, "expert rows: null pointer");
  return lo::expert_rows_impl(xq, xs, 0, row_expert, row_weight, w1, w2, w1_scale, w2_scale, T, E_local, H, I, out,
                              workspace, workspace_bytes, status, stream);
}

extern "C" size_t lo_expert_rows_packed_workspace_bytes(int64_t T, int E_local, int64_t H, int64_t I) {
  using namespace lo;
  return carve_fused(nullptr, T, E_local, 1, H, I).bytes + 2 * (size_t)round_up(T * 4, ALIGN_BYTES) +
         (size_t)round_up(T * 8, ALIGN_BYTES);
}

namespace lo {
namespace {
int expert_rows_packed_impl(const uint8_t *packed, int64_t T, const int8_t *w1, const int8_t *w2, const float *w1_scale,
                            const float *w2_scale, int E_local, int64_t H, int64_t I, void *out, const int32_t *seg_first,
                            const int64_t *seg_ret, int world, void *workspace, size_t workspace_bytes, int32_t *status,
                            void *stream) {
  LO_REQUIRE(T >= 0 && E_local >= 1 && H % 128 == 0 && I % 128 == 0, "expert rows (packed): bad shape");
  if (T == 0) return LO_OK;
  LO_REQUIRE(packed && workspace, "expert rows (packed): null pointer");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 15) == 0, "expert rows (packed): records must be 16-byte aligned");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & (ALIGN_BYTES - 1)) == 0, "expert rows (packed): workspace must be 256-byte aligned");
  const size_t fused_bytes = carve_fused(nullptr, T, E_local, 1, H, I).bytes;
  const size_t meta_bytes = (size_t)round_up(T * 4, ALIGN_BYTES);
  const size_t table_bytes = (size_t)round_up(T * 8, ALIGN_BYTES);
  LO_REQUIRE(workspace_bytes >= fused_bytes + 2 * meta_bytes + table_bytes,
             "expert rows (packed): workspace of %zu bytes, %zu needed", workspace_bytes, fused_bytes + 2 * meta_bytes + table_bytes);
  uint8_t *ws = static_cast<uint8_t *>(workspace);
  int32_t *row_expert = reinterpret_cast<int32_t *>(ws + fused_bytes);
  float *row_weight = reinterpret_cast<float *>(ws + fused_bytes + meta_bytes);
  int64_t *row_dst = seg_ret ? reinterpret_cast<int64_t *>(ws + fused_bytes + 2 * meta_bytes) : nullptr;
  const int64_t stride = lo_ep_dispatch_row_bytes(H);
  int rc = launch_ep_unpack_meta(packed, T, stride, H + 4 * (H / 128), row_expert, row_weight, static_cast<cudaStream_t>(stream),
                                 seg_first, seg_ret, world, 2 * H, row_dst);
  if (rc != LO_OK) return rc;
  return expert_rows_impl(reinterpret_cast<const int8_t *>(packed), nullptr, stride, row_expert, row_weight, w1, w2, w1_scale,
                          w2_scale, T, E_local, H, I, out, workspace, fused_bytes, status, stream, row_dst);
}
}  // namespace
}  // namespace lo

extern "C" int lo_expert_rows_block_int8_packed(const uint8_t *packed, int64_t T, const int8_t *w1, const int8_t *w2,
                                                const float *w1_scale, const float *w2_scale, int E_local, int64_t H,
                                                int64_t I, void *out, void *workspace, size_t workspace_bytes,
                                                int32_t *status, void *stream) {
  using namespace lo;
  LO_REQUIRE(out != nullptr || T == 0, "expert rows (packed): null pointer");
  return expert_rows_packed_impl(packed, T, w1, w2, w1_scale, w2_scale, E_local, H, I, out, nullptr, nullptr, 0, workspace,
                                 workspace_bytes, status, stream);
}

extern "C" int lo_expert_rows_block_int8_packed_put(const uint8_t *packed, int64_t T, const int8_t *w1, const int8_t *w2,
                                                    const float *w1_scale, const float *w2_scale, int E_local, int64_t H,
                                                    int64_t I, const int32_t *seg_first, const int64_t *seg_ret, int world,
                                                    void *workspace, size_t workspace_bytes, int32_t *status, void *stream) {
  using namespace lo;
  LO_REQUIRE(world >= 1 && world <= 1024 && (T == 0 || (seg_first && seg_ret)), "expert rows (put): bad return route");
  return expert_rows_packed_impl(packed, T, w1, w2, w1_scale, w2_scale, E_local, H, I, nullptr, seg_first, seg_ret, world,
                                 workspace, workspace_bytes, status, stream);
}

// ---------------------------------------------------------------------------
// Dense block-INT8 linear: the grouped GEMM with a single "expert" that owns every row.
// ---------------------------------------------------------------------------
namespace lo {
namespace {
__global__ void linear_plan_kernel(int64_t M, int32_t *__restrict__ sorted_ids, Chunk *__restrict__ chunks,
                                   int32_t *__restrict__ num_chunks) {
  const int64_t n_chunks = (M + 127) / 128;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M; i += (int64_t)gridDim.x * blockDim.x)
    sorted_ids[i] = (int32_t)i;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks; c += (int64_t)gridDim.x * blockDim.x) {
    Chunk ch;
    ch.expert = 0;
    ch.row0 = (int32_t)(c * 128);
    ch.rows = (int32_t)(M - c * 128 < 128 ? M - c * 128 : 128);
    ch.pad = 0;
    chunks[c] = ch;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *num_chunks = (int32_t)n_chunks;
}
struct LinearWs {
  int32_t *num_chunks;
  int32_t *sorted_ids;
  Chunk *chunks;
  size_t bytes;
};
LinearWs carve_linear(void *ws, int64_t M) {
  LinearWs W;
  Carver c(ws);
  W.num_chunks = c.take<int32_t>(64);
  W.sorted_ids = c.take<int32_t>(M);
  W.chunks = c.take<Chunk>((M + 127) / 128 + 1);
  W.bytes = c.off;
  return W;
}
}  // namespace
}  // namespace lo

extern "C" size_t lo_block_int8_linear_workspace_bytes(int64_t M) { return M <= 0 ? 0 : lo::carve_linear(nullptr, M).bytes; }

extern "C" int lo_block_int8_linear(const int8_t *A, const float *a_scale, const int8_t *B, const float *b_scale,
                                    int64_t M, int64_t N, int64_t K, void *C, void *workspace, size_t workspace_bytes,
                                    int32_t *status, void *stream) {
  using namespace lo;
  LO_REQUIRE(M >= 0 && N >= 1 && K >= 128 && K % 128 == 0, "block int8 linear: bad shape (K must be a multiple of 128)");
  if (M == 0) return LO_OK;
  LO_REQUIRE(A && a_scale && B && b_scale && C && workspace, "block int8 linear: null pointer");
  LO_REQUIRE(M < (1LL << 30), "block int8 linear: too many rows");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & (ALIGN_BYTES - 1)) == 0, "block int8 linear: workspace must be 256-byte aligned");
  LinearWs W = carve_linear(workspace, M);
  LO_REQUIRE(workspace_bytes >= W.bytes, "block int8 linear: workspace of %zu bytes, %zu needed", workspace_bytes, W.bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = (int)(ceil_div(M, 256) > 1024 ? 1024 : ceil_div(M, 256));
  linear_plan_kernel<<<blocks, 256, 0, st>>>(M, W.sorted_ids, W.chunks, W.num_chunks);
  LO_LAUNCH_OK("linear_plan_kernel");
  GemmArgs g{};
  g.A = A; g.a_scale = a_scale; g.rows_a = M; g.max_chunk_rows = (int)(M < 128 ? M : 128);
  g.B = B; g.b_scale = b_scale; g.E = 1;
  g.n_rows_per_expert = N; g.n_store = N; g.K = K; g.n_tiles = (int)ceil_div(N, 128);
  g.sorted_ids = W.sorted_ids; g.numel_valid = M;
  g.chunks = W.chunks; g.num_chunks = W.num_chunks;
  g.C = static_cast<__nv_bfloat16 *>(C);
  g.weight_mode = LO_WEIGHT_NONE; g.status = status;
  return launch_grouped_gemm(GEMM_SINGLE, g, st);
}
