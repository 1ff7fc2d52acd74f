// Top-k reduction (moe_sum) and the expert-parallel local permutation kernels
// (ep_scatter / ep_build_m_indices / ep_gather).  All are streaming,
// HBM-bound kernels: 16-byte vector accesses, fp32 accumulation.
#include "common.h"
#include <cooperative_groups.h>

namespace lo {
namespace {

template <typename T> struct Vec8;   // 8 elements of T
template <> struct Vec8<__nv_bfloat16> {
  uint4 raw;
  __device__ __forceinline__ void to_float(float (&f)[8]) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ void from_float(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t *>(&p);
    }
    raw = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Vec8<__half> {
  uint4 raw;
  __device__ __forceinline__ void to_float(float (&f)[8]) const {
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 v = __half22float2(h[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
  __device__ __forceinline__ void from_float(const float (&f)[8]) {
    __half2 *h = reinterpret_cast<__half2 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  }
};
template <> struct Vec8<float> {
  float4 a, b;
  __device__ __forceinline__ void to_float(float (&f)[8]) const {
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  __device__ __forceinline__ void from_float(const float (&f)[8]) {
    a = make_float4(f[0], f[1], f[2], f[3]);
    b = make_float4(f[4], f[5], f[6], f[7]);
  }
};

// skip rule of one (token, slot):
//   mask     : optional bool [M, topk]
//   ids/map  : optional routing ids + expert_map; the slot is skipped when its expert is not local
template <typename T, typename IdT>
__global__ void __launch_bounds__(256) moe_sum_kernel(const T *__restrict__ in, T *__restrict__ out,
                                                      const T *__restrict__ bias, int64_t M, int topk, int64_t H8,
                                                      float factor, const uint8_t *__restrict__ mask,
                                                      const int32_t *__restrict__ num_local_tokens,
                                                      const IdT *__restrict__ ids, const int32_t *__restrict__ expert_map,
                                                      int num_experts, int num_local) {
  using V = Vec8<T>;
  const int64_t t = blockIdx.y;
  dependency_wait();            // the rows come from the kernel before this one
  if (num_local_tokens && t >= *num_local_tokens) return;
  const V *in_v = reinterpret_cast<const V *>(in) + t * topk * H8;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < H8; c += (int64_t)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < topk; ++j) {
      if (mask && !mask[t * topk + j]) continue;
      if (ids) {
        // the rule of the alignment kernel (load_expert): an id outside [0, num_experts), or one that maps
        // outside the local experts, was dropped there and its row was never written
        const long long e = (long long)ids[t * topk + j];
        if (e < 0 || e >= num_experts) continue;
        if (expert_map) {
          const int m = expert_map[e];
          if (m < 0 || m >= num_local) continue;
        }
      }
      float f[8];
      in_v[(int64_t)j * H8 + c].to_float(f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    if (bias) {
      float b[8];
      reinterpret_cast<const V *>(bias)[t * H8 + c].to_float(b);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = acc[i] * factor + b[i];
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = acc[i] * factor;
    }
    V o;
    o.from_float(acc);
    reinterpret_cast<V *>(out)[t * H8 + c] = o;
  }
}

template <typename T, typename IdT>
int launch_sum(const void *in, void *out, const void *bias, int64_t M, int topk, int64_t H, float factor,
               const uint8_t *mask, const int32_t *nlt, const void *ids, const int32_t *expert_map,
               cudaStream_t st, int num_experts = 0x7fffffff, int num_local = 0x7fffffff) {
  const int64_t H8 = H / 8;
  dim3 grid((unsigned)(ceil_div(H8, 256) > 65535 ? 65535 : ceil_div(H8, 256)), (unsigned)M);
  LO_CUDA_OK(launch_dependent(moe_sum_kernel<T, IdT>, grid, dim3(256), 0, st, static_cast<const T *>(in),
                              static_cast<T *>(out), static_cast<const T *>(bias), M, topk, H8, factor, mask, nlt,
                              static_cast<const IdT *>(ids), expert_map, num_experts, num_local));
  return LO_OK;
}

// ---------------------------------------------------------------------------
// Expert-parallel local permutation.
// ---------------------------------------------------------------------------

template <typename IdT>
__device__ __forceinline__ int local_expert(const IdT *ids, int64_t i, const int32_t *expert_map, int local_E) {
  long long e = (long long)ids[i];
  if (e < 0) return -1;
  if (expert_map) e = expert_map[e];
  if (e < 0 || e >= local_E) return -1;
  return (int)e;
}

// Aligned exclusive offsets from the per-expert counts, m_indices fill, and the stable destination row of
// every (token, slot) -> inv_perm.  Same scheme as the alignment kernels: per-warp histograms, stable rank
// from peer masks.  Runs as one CTA or, for many ids, as a cluster of EP_PLAN_CLUSTER CTAs that take
// consecutive slices of the ids and exchange their per-expert counts through distributed shared memory.
constexpr int EP_PLAN_CLUSTER = 8;
constexpr int64_t EP_PLAN_CLUSTER_MIN_IDS = 8192;

template <typename IdT>
__global__ void __launch_bounds__(1024) ep_plan_kernel(const IdT *__restrict__ ids, int64_t numel,
                                                       const int32_t *__restrict__ expert_map,
                                                       const int32_t *__restrict__ counts_in, int local_E,
                                                       int alignment, int32_t *__restrict__ m_indices, int64_t rows,
                                                       int32_t *__restrict__ inv_perm, int32_t *__restrict__ counts_out) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks();      // 1 for a plain launch
  const int r = (int)cluster.block_rank();
  extern __shared__ int32_t smem[];
  int32_t *hist = smem;                 // [32][local_E]
  int32_t *off = smem + 32 * local_E;   // [local_E + 1]
  int32_t *cnt = off + local_E + 1;     // [local_E] ids per expert, whole input (or the caller's counts)
  int32_t *cta_cnt = cnt + local_E;     // [local_E] ids per expert in this CTA's slice
  int32_t *before = cta_cnt + local_E;  // [local_E] ids per expert in lower-ranked CTAs
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < 32 * local_E; i += blockDim.x) hist[i] = 0;
  for (int64_t i = (int64_t)r * blockDim.x + tid; i < rows; i += (int64_t)C * blockDim.x) m_indices[i] = -1;
  __syncthreads();
  int64_t cta_len = (numel + C - 1) / C;
  cta_len = (cta_len + 31) / 32 * 32;
  const int64_t cta_begin = (int64_t)r * cta_len;
  const int64_t cta_end = cta_begin + cta_len < numel ? cta_begin + cta_len : numel;
  int64_t seg_len = (cta_len + 31) / 32;
  seg_len = (seg_len + 31) / 32 * 32;
  const int64_t seg_begin = cta_begin + (int64_t)warp * seg_len;
  const int64_t seg_end = seg_begin + seg_len < cta_end ? seg_begin + seg_len : cta_end;
  int32_t *my_hist = hist + warp * local_E;
  // bits that distinguish the local expert ids, or 0 = use the match instruction (few steps per warp)
  const int id_bits = seg_len >= 256 ? 32 - __clz(local_E > 1 ? local_E - 1 : 1) : 0;
  for (int64_t base = seg_begin; base < seg_end; base += 32) {
    const int64_t i = base + lane;
    const int e = i < seg_end ? local_expert<IdT>(ids, i, expert_map, local_E) : -1;
    if (e >= 0) atomicAdd(&my_hist[e], 1);      // counting pass: order does not matter
  }
  __syncthreads();
  for (int e = tid; e < local_E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = hist[w * local_E + e];
      hist[w * local_E + e] = run;
      run += c;
    }
    cta_cnt[e] = run;
  }
  cluster.sync();      // counts of every CTA published, m_indices cleared everywhere
  for (int e = tid; e < local_E; e += blockDim.x) {
    int total = 0, lower = 0;
    for (int rr = 0; rr < C; ++rr) {
      const int v = cluster.map_shared_rank(cta_cnt, rr)[e];
      total += v;
      if (rr < r) lower += v;
    }
    cnt[e] = counts_in ? counts_in[e] : total;
    before[e] = lower;
    if (counts_out != nullptr && r == 0) counts_out[e] = total;
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < local_E; ++e) {
      off[e] = run;
      run += (cnt[e] + alignment - 1) / alignment * alignment;
    }
    off[local_E] = run;
  }
  __syncthreads();
  // expert id of every row: the CTAs share the experts
  for (int e = r * 32 + warp; e < local_E; e += C * 32)
    for (int q = lane; q < cnt[e]; q += 32)
      if (off[e] + q < rows) m_indices[off[e] + q] = e;
  if (inv_perm != nullptr) {
    for (int64_t base = seg_begin; base < seg_end; base += 32) {
      const int64_t i = base + lane;
      const int e = i < seg_end ? local_expert<IdT>(ids, i, expert_map, local_E) : -1;
      const unsigned peers = peers_of(e, id_bits);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      int prior = 0;
      if (e >= 0) prior = my_hist[e];
      __syncwarp();
      if (i < seg_end) inv_perm[i] = e >= 0 ? off[e] + before[e] + prior + rank : -1;
      if (e >= 0 && lane == (__ffs(peers) - 1)) my_hist[e] = prior + __popc(peers);
      __syncwarp();
    }
  }
  cluster.sync();      // no CTA leaves while another may still read its counts
}

template <typename IdT>
int launch_ep_plan(const void *ids, int64_t numel, const int32_t *expert_map, const int32_t *counts_in, int local_E,
                   int alignment, int32_t *m_indices, int64_t rows, int32_t *inv_perm, cudaStream_t st,
                   int32_t *counts_out = nullptr) {
  const size_t smem = sizeof(int32_t) * (36 * (size_t)local_E + 1);
  LO_CUDA_OK(cudaFuncSetAttribute(ep_plan_kernel<IdT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const IdT *idp = static_cast<const IdT *>(ids);
  if (numel >= EP_PLAN_CLUSTER_MIN_IDS) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(EP_PLAN_CLUSTER, 1, 1);
    cfg.blockDim = dim3(1024, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = EP_PLAN_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    LO_CUDA_OK(cudaLaunchKernelEx(&cfg, ep_plan_kernel<IdT>, idp, numel, expert_map, counts_in, local_E, alignment,
                                  m_indices, rows, inv_perm, counts_out));
    return LO_OK;
  }
  ep_plan_kernel<IdT><<<1, 1024, smem, st>>>(idp, numel, expert_map, counts_in, local_E, alignment, m_indices, rows, inv_perm, counts_out);
  LO_LAUNCH_OK("ep_plan_kernel");
  return LO_OK;
}

// One CTA per (token, slot): copy the int8 row and its scales to inv_perm[token, slot].
__global__ void __launch_bounds__(128) ep_copy_rows_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as,
                                                           int scale_cols, const int32_t *__restrict__ inv_perm,
                                                           int8_t *__restrict__ aq_out, float *__restrict__ as_out,
                                                           int k, int64_t H, int64_t rows) {
  const int64_t flat = blockIdx.x;
  const int32_t dst = inv_perm[flat];
  if (dst < 0 || dst >= rows) return;
  const int64_t t = flat / k;
  const uint4 *src = reinterpret_cast<const uint4 *>(aq + t * H);
  uint4 *d = reinterpret_cast<uint4 *>(aq_out + (int64_t)dst * H);
  for (int64_t c = threadIdx.x; c < H / 16; c += blockDim.x) d[c] = src[c];
  for (int c = threadIdx.x; c < scale_cols; c += blockDim.x) as_out[(int64_t)dst * scale_cols + c] = as[t * scale_cols + c];
}

// Dispatch payload of expert parallelism, one CTA per (token, slot): the token's int8 row, its group scales, the
// slot's expert id on the destination rank and its routed weight, as ONE record of `stride` bytes at row
// inv_perm[token, slot] of the send buffer (rows grouped by destination rank), so that a step needs a single
// all-to-all for everything the expert side wants.
template <typename IdT>
__global__ void __launch_bounds__(128) ep_pack_rows_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as,
                                                           const IdT *__restrict__ ids, const float *__restrict__ w,
                                                           const int32_t *__restrict__ inv_perm, uint8_t *__restrict__ out,
                                                           int k, int64_t H, int G, int64_t stride, int experts_per_rank,
                                                           int64_t rows) {
  const int64_t flat = blockIdx.x;
  const int32_t dst = inv_perm[flat];
  if (dst < 0 || dst >= rows) return;
  const int64_t t = flat / k;
  uint8_t *rec = out + (int64_t)dst * stride;
  const uint4 *src = reinterpret_cast<const uint4 *>(aq + t * H);
  uint4 *d = reinterpret_cast<uint4 *>(rec);
  for (int64_t c = threadIdx.x; c < H / 16; c += blockDim.x) d[c] = src[c];
  float *sc = reinterpret_cast<float *>(rec + H);
  for (int c = threadIdx.x; c < G; c += blockDim.x) sc[c] = as[t * G + c];
  if (threadIdx.x == 0) {
    reinterpret_cast<int32_t *>(rec + H + 4 * (int64_t)G)[0] = (int32_t)((long long)ids[flat] % experts_per_rank);
    reinterpret_cast<float *>(rec + H + 4 * (int64_t)G)[1] = w[flat];
  }
}

// The same record, stored straight into the destination rank's receive buffer: seg_dst[d] is the address (in this
// process's address space: local memory or a peer mapping) where this rank's run of records for rank d begins,
// seg_first[d] the packed position of the run's first record.  Plain 16-byte stores; nothing is read from a peer.
template <typename IdT>
__global__ void __launch_bounds__(128) ep_put_rows_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as,
                                                          const IdT *__restrict__ ids, const float *__restrict__ w,
                                                          const int32_t *__restrict__ rank_of_expert,
                                                          const int32_t *__restrict__ inv_perm,
                                                          const int32_t *__restrict__ seg_first,
                                                          const int64_t *__restrict__ seg_dst, int world, int k, int64_t H,
                                                          int G, int64_t stride, int experts_per_rank, int64_t rows) {
  const int64_t flat = blockIdx.x;
  const int32_t pos = inv_perm[flat];
  if (pos < 0 || pos >= rows) return;
  const long long e = (long long)ids[flat];
  const int d = rank_of_expert[e];
  if (d < 0 || d >= world || seg_dst[d] == 0 || pos < seg_first[d]) return;
  const int64_t t = flat / k;
  uint8_t *rec = reinterpret_cast<uint8_t *>(seg_dst[d]) + (int64_t)(pos - seg_first[d]) * stride;
  const uint4 *src = reinterpret_cast<const uint4 *>(aq + t * H);
  uint4 *dp = reinterpret_cast<uint4 *>(rec);
  for (int64_t c = threadIdx.x; c < H / 16; c += blockDim.x) dp[c] = src[c];
  float *sc = reinterpret_cast<float *>(rec + H);
  for (int c = threadIdx.x; c < G; c += blockDim.x) sc[c] = as[t * G + c];
  if (threadIdx.x == 0) {
    reinterpret_cast<int32_t *>(rec + H + 4 * (int64_t)G)[0] = (int32_t)(e % experts_per_rank);
    reinterpret_cast<float *>(rec + H + 4 * (int64_t)G)[1] = w[flat];
  }
}

// Expert id and routed weight of every received record into contiguous arrays (the alignment kernel wants the ids
// as one array).
__global__ void __launch_bounds__(256) ep_unpack_meta_kernel(const uint8_t *__restrict__ packed, int64_t rows, int64_t stride,
                                                             int64_t meta_off, int32_t *__restrict__ row_expert,
                                                             float *__restrict__ row_weight,
                                                             const int32_t *__restrict__ seg_first,
                                                             const int64_t *__restrict__ seg_ret, int world,
                                                             int64_t ret_row_bytes, int64_t *__restrict__ row_dst) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const uint8_t *rec = packed + r * stride + meta_off;
  row_expert[r] = reinterpret_cast<const int32_t *>(rec)[0];
  row_weight[r] = reinterpret_cast<const float *>(rec)[1];
  if (row_dst != nullptr) {
    // Return route of the row: record r belongs to the run of source rank s with seg_first[s] <= r < seg_first[s + 1]
    // and goes back to seg_ret[s] + (r - seg_first[s]) rows (an address in rank s's return buffer).  A row outside
    // every run, or of a run without an address, gets 0 = "do not store".
    int64_t dst = 0;
    for (int s = 0; s < world; ++s)
      if (r >= seg_first[s] && r < seg_first[s + 1] && seg_ret[s] != 0) dst = seg_ret[s] + (r - seg_first[s]) * ret_row_bytes;
    row_dst[r] = dst;
  }
}

template <typename IdT>
__global__ void __launch_bounds__(256) ep_gather_kernel(const __nv_bfloat16 *__restrict__ a, const IdT *__restrict__ ids,
                                                        const float *__restrict__ w, const int32_t *__restrict__ inv_perm,
                                                        const int32_t *__restrict__ expert_map,
                                                        __nv_bfloat16 *__restrict__ out, int k, int64_t H8) {
  using V = Vec8<__nv_bfloat16>;
  const int64_t t = blockIdx.y;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < H8; c += (int64_t)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      // a slot that the scatter dropped has no row (and its id may lie outside the map): look at that first
      const int32_t r = inv_perm[t * k + j];
      if (r < 0) continue;
      const long long e = (long long)ids[t * k + j];
      if (e < 0 || (expert_map && expert_map[e] < 0)) continue;
      const float wj = w[t * k + j];
      float f[8];
      reinterpret_cast<const V *>(a)[(int64_t)r * H8 + c].to_float(f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(wj, f[i], acc[i]);
    }
    V o;
    o.from_float(acc);
    reinterpret_cast<V *>(out)[t * H8 + c] = o;
  }
}

// One CTA per sorted position: copy the int8 row and its scales of token sorted_ids[pos] / top_k.
__global__ void __launch_bounds__(128) permute_rows_kernel(const int8_t *__restrict__ A, const float *__restrict__ a_scale,
                                                           int64_t rows_a, int64_t K, const int32_t *__restrict__ sorted_ids,
                                                           const int32_t *__restrict__ num_tokens_post_pad,
                                                           int64_t numel_valid, int top_k, int64_t kb,
                                                           int8_t *__restrict__ A_sorted,
                                                           float *__restrict__ a_scale_sorted, int64_t a_stride) {
  const int64_t pos = blockIdx.x;
  if (pos >= *num_tokens_post_pad) return;
  const int32_t sid = sorted_ids[pos];
  if (sid < 0 || sid >= numel_valid) return;
  const int64_t row = sid / top_k;
  if (row >= rows_a) return;
  // a_stride: bytes between two source rows (K for a plain matrix); without a scale array the scales follow the
  // row inside its record
  const uint4 *src = reinterpret_cast<const uint4 *>(A + row * a_stride);
  const float *src_s = a_scale ? a_scale + row * kb : reinterpret_cast<const float *>(A + row * a_stride + K);
  uint4 *dst = reinterpret_cast<uint4 *>(A_sorted + pos * K);
  for (int64_t c = threadIdx.x; c < K / 16; c += blockDim.x) dst[c] = src[c];
  for (int64_t c = threadIdx.x; c < kb; c += blockDim.x) a_scale_sorted[pos * kb + c] = src_s[c];
}

}  // namespace

int launch_permute_rows(const int8_t *A, const float *a_scale, int64_t rows_a, int64_t K, const int32_t *sorted_ids,
                        int64_t sorted_capacity, const int32_t *num_tokens_post_pad, int64_t numel_valid, int top_k,
                        int8_t *A_sorted, float *a_scale_sorted, cudaStream_t stream, int64_t scales_per_row,
                        int64_t a_stride) {
  if (sorted_capacity <= 0) return LO_OK;
  LO_REQUIRE(sorted_capacity <= 0x7fffffffLL, "permute rows: too many positions");
  permute_rows_kernel<<<(unsigned)sorted_capacity, 128, 0, stream>>>(A, a_scale, rows_a, K, sorted_ids, num_tokens_post_pad,
                                                                     numel_valid, top_k,
                                                                     scales_per_row > 0 ? scales_per_row : K / 128, A_sorted,
                                                                     a_scale_sorted, a_stride > 0 ? a_stride : K);
  LO_LAUNCH_OK("permute_rows_kernel");
  return LO_OK;
}

int launch_ep_unpack_meta(const uint8_t *packed, int64_t rows, int64_t stride, int64_t meta_off, int32_t *row_expert,
                          float *row_weight, cudaStream_t stream, const int32_t *seg_first, const int64_t *seg_ret,
                          int world, int64_t ret_row_bytes, int64_t *row_dst) {
  if (rows <= 0) return LO_OK;
  ep_unpack_meta_kernel<<<(unsigned)ceil_div(rows, 256), 256, 0, stream>>>(packed, rows, stride, meta_off, row_expert, row_weight,
                                                                          seg_first, seg_ret, world, ret_row_bytes, row_dst);
  LO_LAUNCH_OK("ep_unpack_meta_kernel");
  return LO_OK;
}

int launch_moe_sum_masked(const __nv_bfloat16 *in, __nv_bfloat16 *out, const __nv_bfloat16 *bias, int64_t M,
                          int topk, int64_t H, float factor, const void *topk_ids, int ids_dtype,
                          const int32_t *expert_map, int num_experts, int num_local, cudaStream_t stream) {
  if (M == 0) return LO_OK;
  if (ids_dtype == LO_I64)
    return launch_sum<__nv_bfloat16, int64_t>(in, out, bias, M, topk, H, factor, nullptr, nullptr, topk_ids, expert_map, stream,
                                              num_experts, num_local);
  return launch_sum<__nv_bfloat16, int32_t>(in, out, bias, M, topk, H, factor, nullptr, nullptr, topk_ids, expert_map, stream,
                                            num_experts, num_local);
}

}  // namespace lo

extern "C" int lo_moe_sum(const void *in, void *out, const void *bias, int dtype, int64_t M, int topk, int64_t H,
                          float factor, const uint8_t *expert_mask, const int32_t *num_local_tokens, void *stream) {
  using namespace lo;
  LO_REQUIRE(M >= 0 && topk >= 1 && H >= 0, "moe_sum: bad shape");
  if (M == 0 || H == 0) return LO_OK;
  LO_REQUIRE(in && out, "moe_sum: null pointer");
  LO_REQUIRE(H % 8 == 0, "moe_sum: hidden size %lld is not a multiple of 8", (long long)H);
  LO_REQUIRE(M <= 0x7fffffffLL, "moe_sum: too many tokens");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case LO_BF16: return launch_sum<__nv_bfloat16, int32_t>(in, out, bias, M, topk, H, factor, expert_mask, num_local_tokens, nullptr, nullptr, st);
    case LO_F16: return launch_sum<__half, int32_t>(in, out, bias, M, topk, H, factor, expert_mask, num_local_tokens, nullptr, nullptr, st);
    case LO_F32: return launch_sum<float, int32_t>(in, out, bias, M, topk, H, factor, expert_mask, num_local_tokens, nullptr, nullptr, st);
    default: return fail(LO_ERR_UNSUPPORTED, "moe_sum: unsupported dtype code %d", dtype);
  }
}

extern "C" int lo_ep_build_m_indices(const void *topk_ids, int ids_dtype, int64_t numel, int32_t *m_indices,
                                     int64_t rows, int local_num_experts, int alignment, void *stream) {
  using namespace lo;
  LO_REQUIRE(local_num_experts >= 1 && local_num_experts <= 1024, "ep_build_m_indices: local_num_experts out of range");
  LO_REQUIRE(alignment >= 1 && m_indices && (topk_ids || numel == 0), "ep_build_m_indices: bad argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_dtype == LO_I64)
    return launch_ep_plan<int64_t>(topk_ids, numel, nullptr, nullptr, local_num_experts, alignment, m_indices, rows, nullptr, st);
  if (ids_dtype == LO_I32)
    return launch_ep_plan<int32_t>(topk_ids, numel, nullptr, nullptr, local_num_experts, alignment, m_indices, rows, nullptr, st);
  return fail(LO_ERR_UNSUPPORTED, "ep_build_m_indices: unsupported id dtype code %d", ids_dtype);
}

extern "C" int lo_ep_scatter(const int8_t *aq, const float *aq_scale, int scale_cols, const void *topk_ids,
                             int ids_dtype, const int32_t *expert_map, const int32_t *expert_num_tokens,
                             int8_t *aq_out, float *aq_scale_out, int32_t *m_indices, int32_t *inv_perm, int64_t T,
                             int k, int64_t H, int64_t rows, int local_num_experts, int alignment, void *stream) {
  using namespace lo;
  LO_REQUIRE(local_num_experts >= 1 && local_num_experts <= 1024, "ep_scatter: local_num_experts out of range");
  LO_REQUIRE(alignment >= 1 && k >= 1 && T >= 0 && rows >= 0, "ep_scatter: bad shape");
  LO_REQUIRE(H % 16 == 0, "ep_scatter: hidden size %lld is not a multiple of 16", (long long)H);
  LO_REQUIRE(aq && aq_scale && topk_ids && aq_out && aq_scale_out && m_indices && inv_perm, "ep_scatter: null pointer");
  LO_REQUIRE(T * k <= 0x7fffffffLL, "ep_scatter: too many (token, slot) pairs");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc;
  if (ids_dtype == LO_I64)
    rc = launch_ep_plan<int64_t>(topk_ids, T * k, expert_map, expert_num_tokens, local_num_experts, alignment, m_indices, rows, inv_perm, st);
  else if (ids_dtype == LO_I32)
    rc = launch_ep_plan<int32_t>(topk_ids, T * k, expert_map, expert_num_tokens, local_num_experts, alignment, m_indices, rows, inv_perm, st);
  else
    return fail(LO_ERR_UNSUPPORTED, "ep_scatter: unsupported id dtype code %d", ids_dtype);
  if (rc != LO_OK) return rc;
  if (T * k > 0) {
    ep_copy_rows_kernel<<<(unsigned)(T * k), 128, 0, st>>>(aq, aq_scale, scale_cols, inv_perm, aq_out, aq_scale_out, k, H, rows);
    LO_LAUNCH_OK("ep_copy_rows_kernel");
  }
  return LO_OK;
}

extern "C" int64_t lo_ep_dispatch_row_bytes(int64_t H) { return lo::round_up(H + 4 * (H / 128) + 8, 16); }

extern "C" int lo_ep_dispatch_pack(const int8_t *aq, const float *aq_scale, const void *topk_ids, int ids_dtype,
                                   const float *topk_weights, const int32_t *rank_of_expert, int64_t T, int k, int64_t H,
                                   int experts_per_rank, int world, uint8_t *packed, int32_t *dest_rank,
                                   int32_t *inv_perm, int32_t *counts, void *stream) {
  using namespace lo;
  LO_REQUIRE(world >= 1 && world <= 1024 && experts_per_rank >= 1, "ep_dispatch_pack: bad sharding");
  LO_REQUIRE(k >= 1 && T >= 0 && H % 128 == 0, "ep_dispatch_pack: bad shape");
  LO_REQUIRE(aq && aq_scale && topk_ids && topk_weights && rank_of_expert && packed && dest_rank && inv_perm && counts,
             "ep_dispatch_pack: null pointer");
  LO_REQUIRE(T * k <= 0x7fffffffLL, "ep_dispatch_pack: too many (token, slot) pairs");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t rows = T * k;
  int rc;
  if (ids_dtype == LO_I64)
    rc = launch_ep_plan<int64_t>(topk_ids, rows, rank_of_expert, nullptr, world, 1, dest_rank, rows, inv_perm, st, counts);
  else if (ids_dtype == LO_I32)
    rc = launch_ep_plan<int32_t>(topk_ids, rows, rank_of_expert, nullptr, world, 1, dest_rank, rows, inv_perm, st, counts);
  else
    return fail(LO_ERR_UNSUPPORTED, "ep_dispatch_pack: unsupported id dtype code %d", ids_dtype);
  if (rc != LO_OK || rows == 0) return rc;
  const int64_t stride = lo_ep_dispatch_row_bytes(H);
  if (ids_dtype == LO_I64)
    ep_pack_rows_kernel<int64_t><<<(unsigned)rows, 128, 0, st>>>(aq, aq_scale, static_cast<const int64_t *>(topk_ids), topk_weights,
                                                                 inv_perm, packed, k, H, (int)(H / 128), stride, experts_per_rank, rows);
  else
    ep_pack_rows_kernel<int32_t><<<(unsigned)rows, 128, 0, st>>>(aq, aq_scale, static_cast<const int32_t *>(topk_ids), topk_weights,
                                                                 inv_perm, packed, k, H, (int)(H / 128), stride, experts_per_rank, rows);
  LO_LAUNCH_OK("ep_pack_rows_kernel");
  return LO_OK;
}

extern "C" int lo_ep_dispatch_plan(const void *topk_ids, int ids_dtype, const int32_t *rank_of_expert, int64_t T, int k,
                                   int world, int32_t *dest_rank, int32_t *inv_perm, int32_t *counts, void *stream) {
  using namespace lo;
  LO_REQUIRE(world >= 1 && world <= 1024, "ep_dispatch_plan: bad sharding");
  LO_REQUIRE(k >= 1 && T >= 0 && counts != nullptr, "ep_dispatch_plan: bad shape");
  if (T == 0) {      // a rank without tokens sends nothing
    LO_CUDA_OK(cudaMemsetAsync(counts, 0, sizeof(int32_t) * (size_t)world, static_cast<cudaStream_t>(stream)));
    return LO_OK;
  }
  LO_REQUIRE(topk_ids && rank_of_expert && dest_rank && inv_perm, "ep_dispatch_plan: null pointer");
  LO_REQUIRE(T * k <= 0x7fffffffLL, "ep_dispatch_plan: too many (token, slot) pairs");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t rows = T * k;
  if (ids_dtype == LO_I64)
    return launch_ep_plan<int64_t>(topk_ids, rows, rank_of_expert, nullptr, world, 1, dest_rank, rows, inv_perm, st, counts);
  if (ids_dtype == LO_I32)
    return launch_ep_plan<int32_t>(topk_ids, rows, rank_of_expert, nullptr, world, 1, dest_rank, rows, inv_perm, st, counts);
  return fail(LO_ERR_UNSUPPORTED, "ep_dispatch_plan: unsupported id dtype code %d", ids_dtype);
}

extern "C" int lo_ep_dispatch_put(const int8_t *aq, const float *aq_scale, const void *topk_ids, int ids_dtype,
                                  const float *topk_weights, const int32_t *rank_of_expert, const int32_t *inv_perm,
                                  int64_t T, int k, int64_t H, int experts_per_rank, int world, const int32_t *seg_first,
                                  const int64_t *seg_dst, void *stream) {
  using namespace lo;
  LO_REQUIRE(world >= 1 && world <= 1024 && experts_per_rank >= 1, "ep_dispatch_put: bad sharding");
  LO_REQUIRE(k >= 1 && T >= 0 && H % 128 == 0, "ep_dispatch_put: bad shape");
  if (T == 0) return LO_OK;
  LO_REQUIRE(aq && aq_scale && topk_ids && topk_weights && rank_of_expert && inv_perm && seg_first && seg_dst,
             "ep_dispatch_put: null pointer");
  LO_REQUIRE(T * k <= 0x7fffffffLL, "ep_dispatch_put: too many (token, slot) pairs");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t rows = T * k;
  if (rows == 0) return LO_OK;
  const int64_t stride = lo_ep_dispatch_row_bytes(H);
  if (ids_dtype == LO_I64)
    ep_put_rows_kernel<int64_t><<<(unsigned)rows, 128, 0, st>>>(aq, aq_scale, static_cast<const int64_t *>(topk_ids), topk_weights,
                                                                rank_of_expert, inv_perm, seg_first, seg_dst, world, k, H,
                                                                (int)(H / 128), stride, experts_per_rank, rows);
  else if (ids_dtype == LO_I32)
    ep_put_rows_kernel<int32_t><<<(unsigned)rows, 128, 0, st>>>(aq, aq_scale, static_cast<const int32_t *>(topk_ids), topk_weights,
                                                                rank_of_expert, inv_perm, seg_first, seg_dst, world, k, H,
                                                                (int)(H / 128), stride, experts_per_rank, rows);
  else
    return fail(LO_ERR_UNSUPPORTED, "ep_dispatch_put: unsupported id dtype code %d", ids_dtype);
  LO_LAUNCH_OK("ep_put_rows_kernel");
  return LO_OK;
}

extern "C" int lo_ep_gather(const void *a, const void *topk_ids, int ids_dtype, const float *topk_weights,
                            const int32_t *inv_perm, const int32_t *expert_map, void *out, int64_t T, int k,
                            int64_t H, void *stream) {
  using namespace lo;
  LO_REQUIRE(T >= 0 && k >= 1 && H % 8 == 0, "ep_gather: bad shape");
  if (T == 0) return LO_OK;
  LO_REQUIRE(a && topk_ids && topk_weights && inv_perm && out, "ep_gather: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t H8 = H / 8;
  dim3 grid((unsigned)(ceil_div(H8, 256)), (unsigned)T);
  if (ids_dtype == LO_I64)
    ep_gather_kernel<int64_t><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(a), static_cast<const int64_t *>(topk_ids),
                                                   topk_weights, inv_perm, expert_map, static_cast<__nv_bfloat16 *>(out), k, H8);
  else if (ids_dtype == LO_I32)
    ep_gather_kernel<int32_t><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(a), static_cast<const int32_t *>(topk_ids),
                                                   topk_weights, inv_perm, expert_map, static_cast<__nv_bfloat16 *>(out), k, H8);
  else
    return fail(LO_ERR_UNSUPPORTED, "ep_gather: unsupported id dtype code %d", ids_dtype);
  LO_LAUNCH_OK("ep_gather_kernel");
  return LO_OK;
}
