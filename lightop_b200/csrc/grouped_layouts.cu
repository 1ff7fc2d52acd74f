// Per-channel grouped INT8 GEMM on rows that are ALREADY grouped by expert, in the two layouts that
// expert-parallel dispatchers hand over:
//   contiguous: A [M, K]; m_indices[m] names the expert of row m (-1 = padding row); the rows of an expert are
//               consecutive and every 128-row block holds rows of one expert only (the alignment the producer
//               pads to, a multiple of 128), padding rows at the end of the expert's range;
//   masked:     A [E, max_m, K]; only the first masked_m[e] rows of expert e exist.
// Both only need a chunk table for the grouped GEMM kernel: no permutation, output rows = input rows.
#include "common.h"

namespace lo {
namespace {

constexpr int64_t ALIGN_BYTES = 256;

// One warp per 256-row super-block = two 128-row blocks.  A block's expert is the index of its first row, its
// row count the number of rows carrying that index; a block that is full and followed by a block of the same
// expert is merged with it into one chunk of up to 256 rows (one pass over the expert's weights instead of two).
__global__ void contig_plan_kernel(const int32_t *__restrict__ m_indices, int64_t M, int E, Chunk *__restrict__ chunks,
                                   int32_t *__restrict__ num_chunks, int32_t *__restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int64_t sb = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_sb = (M + 255) / 256;
  if (sb >= n_sb) return;
  int32_t ex[2], rows[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int64_t start = sb * 256 + h * 128;
    int32_t e = start < M ? m_indices[start] : -1;
    if (e >= E) e = -1;
    int cnt = 0, foreign = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t r = start + lane + 32 * j;
      const int32_t v = r < M ? m_indices[r] : -1;
      cnt += (e >= 0 && v == e) ? 1 : 0;
      foreign += (v >= 0 && v != e) ? 1 : 0;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
      foreign += __shfl_xor_sync(0xffffffffu, foreign, off);
    }
    if (foreign > 0 && lane == 0 && status) atomicCAS(status, 0, 20);   // layout contract broken: block skipped
    ex[h] = (e >= 0 && foreign == 0) ? e : -1;
    rows[h] = ex[h] >= 0 ? cnt : 0;
  }
  if (lane == 0) {
    Chunk c0, c1;
    c0.pad = c1.pad = 0;
    c0.row0 = (int32_t)(sb * 256);
    c1.row0 = (int32_t)(sb * 256 + 128);
    if (ex[0] >= 0 && ex[0] == ex[1] && rows[0] == 128) {
      c0.expert = ex[0]; c0.rows = 128 + rows[1];
      c1.expert = -1; c1.rows = 0;
    } else {
      c0.expert = rows[0] > 0 ? ex[0] : -1; c0.rows = rows[0];
      c1.expert = rows[1] > 0 ? ex[1] : -1; c1.rows = rows[1];
    }
    chunks[2 * sb] = c0;
    chunks[2 * sb + 1] = c1;
    if (sb == 0) *num_chunks = (int32_t)(2 * n_sb);
  }
}

// One thread per (expert, 256-row block of its max_m rows).
__global__ void masked_plan_kernel(const int32_t *__restrict__ masked_m, int E, int64_t max_m, int blocks_per_expert,
                                   Chunk *__restrict__ chunks, int32_t *__restrict__ num_chunks) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)E * blocks_per_expert) return;
  const int e = (int)(i / blocks_per_expert);
  const int b = (int)(i % blocks_per_expert);
  int64_t valid = masked_m[e];
  valid = valid < 0 ? 0 : (valid > max_m ? max_m : valid);
  int64_t rows = valid - (int64_t)b * 256;
  rows = rows < 0 ? 0 : (rows > 256 ? 256 : rows);
  Chunk c;
  c.expert = rows > 0 ? e : -1;
  c.row0 = (int32_t)(e * max_m + (int64_t)b * 256);
  c.rows = (int32_t)rows;
  c.pad = 0;
  chunks[i] = c;
  if (i == 0) *num_chunks = E * blocks_per_expert;
}

struct PlanWs {
  int32_t *num_chunks;
  Chunk *chunks;
  size_t bytes;
};
PlanWs carve_plan(void *ws, int64_t max_chunks) {
  PlanWs W;
  uint8_t *base = static_cast<uint8_t *>(ws);
  size_t off = 0;
  W.num_chunks = base ? reinterpret_cast<int32_t *>(base) : nullptr;
  off += (size_t)round_up(64 * (int64_t)sizeof(int32_t), ALIGN_BYTES);
  W.chunks = base ? reinterpret_cast<Chunk *>(base + off) : nullptr;
  off += (size_t)round_up((max_chunks + 1) * (int64_t)sizeof(Chunk), ALIGN_BYTES);
  W.bytes = off;
  return W;
}

int run_channel_gemm(const int8_t *A, const float *a_scale, int64_t rows_a, const int8_t *B, const float *b_scale, int E,
                     int64_t N, int64_t K, void *C, const PlanWs &W, int cap, int32_t *status, cudaStream_t st) {
  GemmArgs g{};
  g.A = A; g.a_scale = a_scale; g.rows_a = rows_a; g.max_chunk_rows = cap;
  g.B = B; g.b_scale = b_scale; g.E = E;
  g.n_rows_per_expert = N; g.K = K; g.n_tiles = (int)(N / 128);
  g.sorted_ids = nullptr; g.numel_valid = rows_a;       // output row = input row
  g.chunks = W.chunks; g.num_chunks = W.num_chunks;
  g.C = static_cast<__nv_bfloat16 *>(C);
  g.weight_mode = LO_WEIGHT_NONE; g.status = status;
  return launch_grouped_gemm(GEMM_CHANNEL, g, st);
}

}  // namespace
}  // namespace lo

extern "C" size_t lo_m_grouped_gemm_workspace_bytes(int64_t total_rows, int num_groups) {
  if (total_rows <= 0 || num_groups <= 0) return 0;
  // contiguous: 2 chunks per 256 rows; masked: ceil(max_m / 256) per group <= rows / 256 + groups
  return lo::carve_plan(nullptr, 2 * ((total_rows + 255) / 256) + num_groups).bytes;
}

extern "C" int lo_m_grouped_w8a8_gemm_nt_contig(const int8_t *A, const float *a_scale, const int8_t *B,
                                                const float *b_scale, void *C, const int32_t *m_indices, int64_t M,
                                                int E, int64_t N, int64_t K, void *workspace, size_t workspace_bytes,
                                                int32_t *status, void *stream) {
  using namespace lo;
  LO_REQUIRE(M >= 0 && E >= 1, "grouped gemm (contiguous): bad shape");
  if (M == 0) return LO_OK;
  LO_REQUIRE(A && a_scale && B && b_scale && C && m_indices && workspace, "grouped gemm (contiguous): null pointer");
  LO_REQUIRE(K % 128 == 0 && N % 128 == 0, "grouped gemm (contiguous): N and K must be multiples of 128");
  LO_REQUIRE(M < (1LL << 31), "grouped gemm (contiguous): too many rows");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & (ALIGN_BYTES - 1)) == 0, "grouped gemm (contiguous): workspace must be 256-byte aligned");
  const int64_t n_sb = (M + 255) / 256;
  PlanWs W = carve_plan(workspace, 2 * n_sb);
  LO_REQUIRE(workspace_bytes >= W.bytes, "grouped gemm (contiguous): workspace of %zu bytes, %zu needed", workspace_bytes, W.bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t threads = n_sb * 32;
  contig_plan_kernel<<<(unsigned)ceil_div(threads, 256), 256, 0, st>>>(m_indices, M, E, W.chunks, W.num_chunks, status);
  LO_LAUNCH_OK("contig_plan_kernel");
  return run_channel_gemm(A, a_scale, M, B, b_scale, E, N, K, C, W, (int)(M < 256 ? M : 256), status, st);
}

extern "C" int lo_m_grouped_w8a8_gemm_nt_masked(const int8_t *A, const float *a_scale, const int8_t *B,
                                                const float *b_scale, void *C, const int32_t *masked_m, int E,
                                                int64_t max_m, int64_t N, int64_t K, void *workspace,
                                                size_t workspace_bytes, int32_t *status, void *stream) {
  using namespace lo;
  LO_REQUIRE(E >= 1 && max_m >= 0, "grouped gemm (masked): bad shape");
  if (max_m == 0) return LO_OK;
  LO_REQUIRE(A && a_scale && B && b_scale && C && masked_m && workspace, "grouped gemm (masked): null pointer");
  LO_REQUIRE(K % 128 == 0 && N % 128 == 0, "grouped gemm (masked): N and K must be multiples of 128");
  LO_REQUIRE((int64_t)E * max_m < (1LL << 31), "grouped gemm (masked): too many rows");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & (ALIGN_BYTES - 1)) == 0, "grouped gemm (masked): workspace must be 256-byte aligned");
  const int bpe = (int)((max_m + 255) / 256);
  PlanWs W = carve_plan(workspace, (int64_t)E * bpe);
  LO_REQUIRE(workspace_bytes >= W.bytes, "grouped gemm (masked): workspace of %zu bytes, %zu needed", workspace_bytes, W.bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  masked_plan_kernel<<<(unsigned)ceil_div((int64_t)E * bpe, 256), 256, 0, st>>>(masked_m, E, max_m, bpe, W.chunks, W.num_chunks);
  LO_LAUNCH_OK("masked_plan_kernel");
  return run_channel_gemm(A, a_scale, (int64_t)E * max_m, B, b_scale, E, N, K, C, W, (int)(max_m < 256 ? max_m : 256), status, st);
}
