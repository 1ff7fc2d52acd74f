// Routing kernels: softmax + top-k selection, and expert alignment
// (histogram + prefix scan + stable scatter) with the grouped-GEMM chunk table.
#include "common.h"
#include <cooperative_groups.h>

namespace lo {
namespace {

// ---------------------------------------------------------------------------
// topk_softmax: one warp per row, experts strided over the lanes (expert =
// lane + 32*i), k rounds of warp arg-max with erase.  Selection is done on the
// logits (softmax is monotonic); ties go to the lower expert id.
// ---------------------------------------------------------------------------

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename IdT> __device__ __forceinline__ void store_id(IdT *p, int v) { *p = (IdT)v; }

template <typename T, typename IdT, int VPL>
__global__ void __launch_bounds__(256) topk_softmax_kernel(const T *__restrict__ gating, int64_t M, int E, int k,
                                                           int renorm, float *__restrict__ weights,
                                                           IdT *__restrict__ ids, int32_t *__restrict__ src_rows) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
  const T *g = gating + row * E;
  float v[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? to_float<T>(g[e]) : -INFINITY;
  }
  // row maximum and softmax denominator over all experts
  float mx = v[0];
#pragma unroll
  for (int i = 1; i < VPL; ++i) mx = fmaxf(mx, v[i]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  float denom = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) denom += (lane + 32 * i < E) ? expf(v[i] - mx) : 0.f;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, off);

  float my_w = 0.f;   // lane j keeps the j-th selected probability
  int my_id = 0;
  float sel_sum = 0.f;
  for (int r = 0; r < k; ++r) {
    float best = v[0];
    int best_e = lane;
#pragma unroll
    for (int i = 1; i < VPL; ++i) {
      if (v[i] > best) { best = v[i]; best_e = lane + 32 * i; }   // strict: keeps the lower id on ties
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    const float p = expf(best - mx) / denom;
    sel_sum += p;
    if (lane == r) { my_w = p; my_id = best_e; }
    // erase the winner in its owner lane
    if ((best_e & 31) == lane) {
      const int slot = best_e >> 5;
#pragma unroll
      for (int i = 0; i < VPL; ++i)
        if (i == slot) v[i] = -INFINITY;
    }
  }
  if (lane < k) {
    const float w = renorm ? my_w / sel_sum : my_w;
    weights[row * k + lane] = w;
    store_id<IdT>(ids + row * k + lane, my_id);
    if (src_rows) src_rows[row * k + lane] = (int32_t)(lane * M + row);
  }
}

template <typename T, typename IdT>
int launch_topk_vpl(const void *gating, int64_t M, int E, int k, int renorm, float *w, void *ids,
                    int32_t *src, cudaStream_t st) {
  const int warps = 8;
  const int64_t blocks = ceil_div(M, warps);
  const T *g = static_cast<const T *>(gating);
  IdT *idp = static_cast<IdT *>(ids);
  const int vpl = (int)ceil_div(E, 32);
#define LO_TOPK_CASE(V)                                                                        \
  topk_softmax_kernel<T, IdT, V><<<(unsigned)blocks, warps * 32, 0, st>>>(g, M, E, k, renorm, w, idp, src)
  if (vpl <= 1) LO_TOPK_CASE(1);
  else if (vpl <= 2) LO_TOPK_CASE(2);
  else if (vpl <= 4) LO_TOPK_CASE(4);
  else if (vpl <= 8) LO_TOPK_CASE(8);
  else if (vpl <= 16) LO_TOPK_CASE(16);
  else LO_TOPK_CASE(32);
#undef LO_TOPK_CASE
  LO_LAUNCH_OK("topk_softmax_kernel");
  return LO_OK;
}

template <typename T>
int launch_topk_ids(const void *gating, int64_t M, int E, int k, int renorm, float *w, void *ids,
                    int ids_dtype, int32_t *src, cudaStream_t st) {
  switch (ids_dtype) {
    case LO_I32: return launch_topk_vpl<T, int32_t>(gating, M, E, k, renorm, w, ids, src, st);
    case LO_U32: return launch_topk_vpl<T, uint32_t>(gating, M, E, k, renorm, w, ids, src, st);
    case LO_I64: return launch_topk_vpl<T, int64_t>(gating, M, E, k, renorm, w, ids, src, st);
    default: return fail(LO_ERR_UNSUPPORTED, "topk_softmax: unsupported index dtype code %d", ids_dtype);
  }
}

// ---------------------------------------------------------------------------
// moe_align_block_size.
//
// One CTA of 32 warps.  The flat id list is cut into 32 contiguous segments,
// one per warp, which the warp walks 32 ids at a time, counting into the
// warp's private histogram row in shared memory.  After an
// exclusive prefix over the warps (per expert) and a block-wide exclusive scan
// of the padded counts (over experts) the warps walk their segments again and
// scatter: position = segment offset of the expert + ids of the same expert in
// earlier warps + ids seen so far by this warp + rank inside the match group.
// That is a stable counting sort, so the order inside an expert is ascending
// flat index, bit-identical run to run.
// ---------------------------------------------------------------------------

constexpr int ALIGN_WARPS = 32;

template <typename IdT>
__device__ __forceinline__ int load_expert(const IdT *ids, int64_t i, int64_t numel, int E,
                                           const int32_t *expert_map, int map_mode) {
  if (i >= numel) return -1;
  long long e = (long long)ids[i];
  if (e < 0 || e >= E) return -1;
  if (map_mode == 1) {
    e = expert_map[e];
    if (e < 0 || e >= E) return -1;
  }
  return (int)e;
}

template <typename IdT>
__global__ void __launch_bounds__(ALIGN_WARPS * 32) align_kernel(
    const IdT *__restrict__ ids, int64_t numel, int E, int block_size, const int32_t *__restrict__ expert_map,
    int map_mode, int32_t *__restrict__ sorted_ids, int64_t sorted_capacity, int32_t *__restrict__ expert_ids,
    int64_t expert_ids_capacity, int32_t *__restrict__ num_tokens_post_pad, Chunk *__restrict__ chunks,
    int32_t *__restrict__ num_chunks, int64_t chunk_capacity, int32_t *__restrict__ inv_pos, int chunk_max) {
  extern __shared__ int32_t smem[];
  int32_t *hist = smem;                       // [ALIGN_WARPS][E]
  int32_t *seg_off = smem + ALIGN_WARPS * E;  // [E + 1] padded exclusive offsets
  int32_t *count = seg_off + (E + 1);         // [E]
  int32_t *chunk_off = count + E;             // [E + 1]
  int32_t *warp_tot = chunk_off + (E + 1);    // [2][32]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  dependency_release();      // the next kernel may get its blocks resident; it waits for this grid before reading

  // warps that get a segment: with few ids (decode) only the first ones, so that the histogram rows to
  // clear and to scan shrink with the input
  const int nw = (int)(numel >= (int64_t)ALIGN_WARPS * 32 ? ALIGN_WARPS : (numel + 31) / 32 > 0 ? (numel + 31) / 32 : 1);
  for (int64_t i = tid; i < sorted_capacity; i += blockDim.x) sorted_ids[i] = (int32_t)numel;
  for (int i = tid; i < nw * E; i += blockDim.x) hist[i] = 0;
  __syncthreads();

  // segment of this warp, a multiple of 32 ids long
  int64_t seg_len = (numel + nw - 1) / nw;
  seg_len = (seg_len + 31) / 32 * 32;
  // bits that distinguish expert ids 0..E-1, or 0 = use the match instruction (see peers_of)
  const int id_bits = seg_len >= 256 ? 32 - __clz(E > 1 ? E - 1 : 1) : 0;
  const int64_t seg_begin = (int64_t)warp * seg_len;
  const int64_t seg_end = seg_begin + seg_len < numel ? seg_begin + seg_len : numel;
  int32_t *my_hist = hist + warp * E;

  // counting pass: order does not matter here, a shared-memory atomic per id is the cheapest way
  for (int64_t base = seg_begin; base < seg_end; base += 32) {
    const int e = load_expert<IdT>(ids, base + lane, seg_end, E, expert_map, map_mode);
    if (e >= 0) atomicAdd(&my_hist[e], 1);
  }
  __syncthreads();

  // per expert: exclusive prefix over the warps, total count
  for (int e = tid; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < nw; ++w) {
      const int c = hist[w * E + e];
      hist[w * E + e] = run;
      run += c;
    }
    count[e] = run;
  }
  __syncthreads();

  // block-wide exclusive scans over experts: padded row counts and 128-row chunk counts.
  // E <= 1024 = blockDim.x, one expert per thread.
  {
    const int c = tid < E ? count[tid] : 0;
    const int padded = (c + block_size - 1) / block_size * block_size;
    const int nch = (c + chunk_max - 1) / chunk_max;
    int a = padded, b = nch;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int ta = __shfl_up_sync(0xffffffffu, a, off);
      const int tb = __shfl_up_sync(0xffffffffu, b, off);
      if (lane >= off) { a += ta; b += tb; }
    }
    if (lane == 31) { warp_tot[warp] = a; warp_tot[32 + warp] = b; }
    __syncthreads();
    if (warp == 0) {
      int ta = warp_tot[lane], tb = warp_tot[32 + lane];
      const int ia = ta, ib = tb;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int ua = __shfl_up_sync(0xffffffffu, ta, off);
        const int ub = __shfl_up_sync(0xffffffffu, tb, off);
        if (lane >= off) { ta += ua; tb += ub; }
      }
      warp_tot[lane] = ta - ia;        // exclusive prefix of the warp totals
      warp_tot[32 + lane] = tb - ib;
    }
    __syncthreads();
    if (tid < E) {
      seg_off[tid] = warp_tot[warp] + a - padded;
      chunk_off[tid] = warp_tot[32 + warp] + b - nch;
      if (tid == E - 1) {
        seg_off[E] = warp_tot[warp] + a;
        chunk_off[E] = warp_tot[32 + warp] + b;
      }
    }
    __syncthreads();
  }
  const int total_padded = seg_off[E];
  if (tid == 0) {
    *num_tokens_post_pad = total_padded;
    if (num_chunks) *num_chunks = chunk_off[E] < chunk_capacity ? chunk_off[E] : (int32_t)chunk_capacity;
  }

  // block -> expert table
  if (expert_ids) {
    const int64_t total_blocks = total_padded / block_size;
    for (int64_t b = total_blocks + tid; b < expert_ids_capacity; b += blockDim.x) expert_ids[b] = -1;
    for (int e = tid; e < E; e += blockDim.x) {
      const int out_e = map_mode == 2 ? expert_map[e] : e;
      for (int b = seg_off[e] / block_size; b < seg_off[e + 1] / block_size; ++b)
        if (b < expert_ids_capacity) expert_ids[b] = out_e;
    }
  }
  // chunk table for the fused path: <=128 consecutive rows of one expert each
  if (chunks) {
    for (int e = tid; e < E; e += blockDim.x) {
      // the rows of an expert are cut into equal chunks (rounded up to the MMA N granule of 16):
      // chunks of one expert then take about the same time and read the weight tiles together
      const int c = count[e];
      const int nch = (c + chunk_max - 1) / chunk_max;
      const int per = nch > 0 ? (((c + nch - 1) / nch) + 15) / 16 * 16 : 0;
      int ci = chunk_off[e];
      for (int r = 0; r < c; r += per, ++ci) {
        if (ci < chunk_capacity) {
          Chunk ch;
          ch.expert = e;
          ch.row0 = seg_off[e] + r;
          ch.rows = c - r < per ? c - r : per;
          ch.pad = (c - r - 1) / per;        // chunks of this expert that follow (their weight tiles are read again soon)
          chunks[ci] = ch;
        }
      }
    }
  }

  // stable scatter
  for (int64_t base = seg_begin; base < seg_end; base += 32) {
    const int e = load_expert<IdT>(ids, base + lane, seg_end, E, expert_map, map_mode);
    const unsigned peers = peers_of(e, id_bits);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int before = 0;
    if (e >= 0) before = my_hist[e];
    __syncwarp();
    if (e >= 0) {
      const int64_t pos = (int64_t)seg_off[e] + before + rank;
      if (pos < sorted_capacity) sorted_ids[pos] = (int32_t)(base + lane);
      if (inv_pos) inv_pos[base + lane] = (int32_t)pos;
      if (lane == (__ffs(peers) - 1)) my_hist[e] = before + __popc(peers);
    } else if (inv_pos && base + lane < seg_end) {
      inv_pos[base + lane] = -1;
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------
// The same alignment for many ids, as a thread-block CLUSTER of ALIGN_CLUSTER CTAs (one launch).
// The single-CTA kernel above is bound by the instruction issue rate of its one SM (about 140
// instructions per warp step over 32 k ids at the prefill size).  Here CTA r of the cluster takes the r-th
// contiguous slice of the ids; the CTAs exchange their per-expert counts through distributed shared
// memory, every CTA repeats the (cheap) scans over experts, and the position of an id is
//   segment offset of its expert + ids of that expert in lower-ranked CTAs + in earlier warps of this
//   CTA + seen so far by this warp + rank inside the warp step,
// i.e. still ascending flat index inside an expert: bit-identical to the single-CTA kernel.
// ---------------------------------------------------------------------------
constexpr int ALIGN_CLUSTER = 8;
constexpr int64_t ALIGN_CLUSTER_MIN_IDS = 8192;   // below this the single CTA is as fast and costs one SM

template <typename IdT>
__global__ void __launch_bounds__(ALIGN_WARPS * 32) align_cluster_kernel(
    const IdT *__restrict__ ids, int64_t numel, int E, int block_size, const int32_t *__restrict__ expert_map,
    int map_mode, int32_t *__restrict__ sorted_ids, int64_t sorted_capacity, int32_t *__restrict__ expert_ids,
    int64_t expert_ids_capacity, int32_t *__restrict__ num_tokens_post_pad, Chunk *__restrict__ chunks,
    int32_t *__restrict__ num_chunks, int64_t chunk_capacity, int32_t *__restrict__ inv_pos, int chunk_max) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks();
  const int r = (int)cluster.block_rank();
  extern __shared__ int32_t smem[];
  int32_t *hist = smem;                       // [ALIGN_WARPS][E] per-warp counts, then exclusive prefixes inside this CTA
  int32_t *seg_off = smem + ALIGN_WARPS * E;  // [E + 1] padded exclusive offsets
  int32_t *count = seg_off + (E + 1);         // [E] ids per expert, whole input
  int32_t *chunk_off = count + E;             // [E + 1]
  int32_t *warp_tot = chunk_off + (E + 1);    // [2][32]
  int32_t *cta_cnt = warp_tot + 64;           // [E] ids per expert in this CTA's slice (read by the other CTAs)
  int32_t *before = cta_cnt + E;              // [E] ids per expert in lower-ranked CTAs

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  dependency_release();
  // sentinel fill: every CTA fills its share
  for (int64_t i = (int64_t)r * blockDim.x + tid; i < sorted_capacity; i += (int64_t)C * blockDim.x) sorted_ids[i] = (int32_t)numel;
  for (int i = tid; i < ALIGN_WARPS * E; i += blockDim.x) hist[i] = 0;
  __syncthreads();

  // slice of this CTA and segment of this warp, both multiples of 32 ids long
  int64_t cta_len = (numel + C - 1) / C;
  cta_len = (cta_len + 31) / 32 * 32;
  const int64_t cta_begin = (int64_t)r * cta_len;
  const int64_t cta_end = cta_begin + cta_len < numel ? cta_begin + cta_len : numel;
  int64_t seg_len = (cta_len + ALIGN_WARPS - 1) / ALIGN_WARPS;
  seg_len = (seg_len + 31) / 32 * 32;
  const int64_t seg_begin = cta_begin + (int64_t)warp * seg_len;
  const int64_t seg_end = seg_begin + seg_len < cta_end ? seg_begin + seg_len : cta_end;
  const int id_bits = seg_len >= 256 ? 32 - __clz(E > 1 ? E - 1 : 1) : 0;
  int32_t *my_hist = hist + warp * E;

  for (int64_t base = seg_begin; base < seg_end; base += 32) {
    const int e = load_expert<IdT>(ids, base + lane, seg_end, E, expert_map, map_mode);
    if (e >= 0) atomicAdd(&my_hist[e], 1);
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < ALIGN_WARPS; ++w) {
      const int c = hist[w * E + e];
      hist[w * E + e] = run;
      run += c;
    }
    cta_cnt[e] = run;
  }
  cluster.sync();      // every CTA's counts are published (and the sentinel fill is complete everywhere)
  for (int e = tid; e < E; e += blockDim.x) {
    int total = 0, lower = 0;
    for (int rr = 0; rr < C; ++rr) {
      const int v = cluster.map_shared_rank(cta_cnt, rr)[e];
      total += v;
      if (rr < r) lower += v;
    }
    count[e] = total;
    before[e] = lower;
  }
  __syncthreads();

  // block-wide exclusive scans over experts (one expert per thread), the same in every CTA
  {
    const int c = tid < E ? count[tid] : 0;
    const int padded = (c + block_size - 1) / block_size * block_size;
    const int nch = (c + chunk_max - 1) / chunk_max;
    int a = padded, b = nch;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int ta = __shfl_up_sync(0xffffffffu, a, off);
      const int tb = __shfl_up_sync(0xffffffffu, b, off);
      if (lane >= off) { a += ta; b += tb; }
    }
    if (lane == 31) { warp_tot[warp] = a; warp_tot[32 + warp] = b; }
    __syncthreads();
    if (warp == 0) {
      int ta = warp_tot[lane], tb = warp_tot[32 + lane];
      const int ia = ta, ib = tb;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int ua = __shfl_up_sync(0xffffffffu, ta, off);
        const int ub = __shfl_up_sync(0xffffffffu, tb, off);
        if (lane >= off) { ta += ua; tb += ub; }
      }
      warp_tot[lane] = ta - ia;
      warp_tot[32 + lane] = tb - ib;
    }
    __syncthreads();
    if (tid < E) {
      seg_off[tid] = warp_tot[warp] + a - padded;
      chunk_off[tid] = warp_tot[32 + warp] + b - nch;
      if (tid == E - 1) {
        seg_off[E] = warp_tot[warp] + a;
        chunk_off[E] = warp_tot[32 + warp] + b;
      }
    }
    __syncthreads();
  }
  const int total_padded = seg_off[E];
  if (r == 0 && tid == 0) {
    *num_tokens_post_pad = total_padded;
    if (num_chunks) *num_chunks = chunk_off[E] < chunk_capacity ? chunk_off[E] : (int32_t)chunk_capacity;
  }
  // block -> expert table and chunk table: CTA r takes the experts e = r, r + C, ...
  if (expert_ids) {
    const int64_t total_blocks = total_padded / block_size;
    for (int64_t b = total_blocks + (int64_t)r * blockDim.x + tid; b < expert_ids_capacity; b += (int64_t)C * blockDim.x) expert_ids[b] = -1;
    for (int e = r + C * tid; e < E; e += C * blockDim.x) {
      const int out_e = map_mode == 2 ? expert_map[e] : e;
      for (int b = seg_off[e] / block_size; b < seg_off[e + 1] / block_size; ++b)
        if (b < expert_ids_capacity) expert_ids[b] = out_e;
    }
  }
  if (chunks) {
    for (int e = r + C * tid; e < E; e += C * blockDim.x) {
      const int c = count[e];
      const int nch = (c + chunk_max - 1) / chunk_max;
      const int per = nch > 0 ? (((c + nch - 1) / nch) + 15) / 16 * 16 : 0;
      int ci = chunk_off[e];
      for (int rr = 0; rr < c; rr += per, ++ci) {
        if (ci < chunk_capacity) {
          Chunk ch;
          ch.expert = e;
          ch.row0 = seg_off[e] + rr;
          ch.rows = c - rr < per ? c - rr : per;
          ch.pad = (c - rr - 1) / per;
          chunks[ci] = ch;
        }
      }
    }
  }

  // stable scatter of this CTA's slice
  for (int64_t base = seg_begin; base < seg_end; base += 32) {
    const int e = load_expert<IdT>(ids, base + lane, seg_end, E, expert_map, map_mode);
    const unsigned peers = peers_of(e, id_bits);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int prior = 0;
    if (e >= 0) prior = my_hist[e];
    __syncwarp();
    if (e >= 0) {
      const int64_t pos = (int64_t)seg_off[e] + before[e] + prior + rank;
      if (pos < sorted_capacity) sorted_ids[pos] = (int32_t)(base + lane);
      if (inv_pos) inv_pos[base + lane] = (int32_t)pos;
      if (lane == (__ffs(peers) - 1)) my_hist[e] = prior + __popc(peers);
    } else if (inv_pos && base + lane < seg_end) {
      inv_pos[base + lane] = -1;
    }
    __syncwarp();
  }
  cluster.sync();      // no CTA leaves while another may still read its counts
}

__global__ void chunks_from_blocks_kernel(const int32_t *__restrict__ expert_ids,
                                          const int32_t *__restrict__ num_tokens_post_pad, int block_size,
                                          int64_t max_blocks, Chunk *__restrict__ chunks,
                                          int32_t *__restrict__ num_chunks) {
  const int64_t total_blocks = min((int64_t)(*num_tokens_post_pad / block_size), max_blocks);
  const int per_block = block_size <= 128 ? 1 : block_size / 128;
  const int rows = block_size <= 128 ? block_size : 128;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_blocks * per_block;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t b = i / per_block;
    Chunk ch;
    ch.expert = expert_ids[b];
    ch.row0 = (int32_t)(b * block_size + (i % per_block) * 128);
    ch.rows = rows;
    ch.pad = 0;
    chunks[i] = ch;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *num_chunks = (int32_t)(total_blocks * per_block);
}


}  // namespace

int launch_align(const void *topk_ids, int ids_dtype, int64_t numel, int num_experts, int block_size,
                 const int32_t *expert_map, int map_mode, int32_t *sorted_ids, int64_t sorted_capacity,
                 int32_t *expert_ids, int64_t expert_ids_capacity, int32_t *num_tokens_post_pad,
                 Chunk *chunks, int32_t *num_chunks, int64_t chunk_capacity, int32_t *inv_pos,
                 int chunk_max, cudaStream_t stream) {
  if (chunk_max != 32 && chunk_max != 64 && chunk_max != 160 && chunk_max != 256) chunk_max = 128;
  LO_REQUIRE(num_experts >= 1 && num_experts <= 1024, "moe_align: num_experts %d outside [1,1024]", num_experts);
  LO_REQUIRE(block_size >= 1, "moe_align: block_size must be positive");
  LO_REQUIRE(numel >= 0 && numel < (1LL << 30), "moe_align: numel out of range");
  LO_REQUIRE(map_mode == 0 || expert_map != nullptr, "moe_align: map_mode %d needs an expert_map", map_mode);
  LO_REQUIRE(sorted_ids && num_tokens_post_pad, "moe_align: null output");
  const size_t smem = sizeof(int32_t) * ((size_t)ALIGN_WARPS * num_experts + 3 * (size_t)num_experts + 2 + 64);
  cudaError_t e;
  if (numel >= ALIGN_CLUSTER_MIN_IDS && (ids_dtype == LO_I32 || ids_dtype == LO_I64)) {
    // many ids: one cluster of ALIGN_CLUSTER CTAs
    const size_t csmem = smem + sizeof(int32_t) * 2 * (size_t)num_experts;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ALIGN_CLUSTER, 1, 1);
    cfg.blockDim = dim3(ALIGN_WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = csmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ALIGN_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (ids_dtype == LO_I32) {
      if (csmem > 48 * 1024)
        LO_CUDA_OK(cudaFuncSetAttribute(align_cluster_kernel<int32_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csmem));
      g_launch_count.fetch_add(1, std::memory_order_relaxed);
      LO_CUDA_OK(cudaLaunchKernelEx(&cfg, align_cluster_kernel<int32_t>, static_cast<const int32_t *>(topk_ids), numel,
                                    num_experts, block_size, expert_map, map_mode, sorted_ids, sorted_capacity, expert_ids,
                                    expert_ids_capacity, num_tokens_post_pad, chunks, num_chunks, chunk_capacity, inv_pos,
                                    chunk_max));
    } else {
      if (csmem > 48 * 1024)
        LO_CUDA_OK(cudaFuncSetAttribute(align_cluster_kernel<int64_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csmem));
      g_launch_count.fetch_add(1, std::memory_order_relaxed);
      LO_CUDA_OK(cudaLaunchKernelEx(&cfg, align_cluster_kernel<int64_t>, static_cast<const int64_t *>(topk_ids), numel,
                                    num_experts, block_size, expert_map, map_mode, sorted_ids, sorted_capacity, expert_ids,
                                    expert_ids_capacity, num_tokens_post_pad, chunks, num_chunks, chunk_capacity, inv_pos,
                                    chunk_max));
    }
    return LO_OK;
  }
  if (ids_dtype == LO_I32) {
    // the opt-in belongs to the (kernel, device) pair: set whenever a launch needs it, whichever device is current
    if (smem > 48 * 1024) {
      e = cudaFuncSetAttribute(align_kernel<int32_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return fail(LO_ERR_CUDA, "moe_align: smem opt-in failed: %s", cudaGetErrorString(e));
    }
    align_kernel<int32_t><<<1, ALIGN_WARPS * 32, smem, stream>>>(
        static_cast<const int32_t *>(topk_ids), numel, num_experts, block_size, expert_map, map_mode, sorted_ids,
        sorted_capacity, expert_ids, expert_ids_capacity, num_tokens_post_pad, chunks, num_chunks, chunk_capacity, inv_pos, chunk_max);
  } else if (ids_dtype == LO_I64) {
    if (smem > 48 * 1024) {
      e = cudaFuncSetAttribute(align_kernel<int64_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return fail(LO_ERR_CUDA, "moe_align: smem opt-in failed: %s", cudaGetErrorString(e));
    }
    align_kernel<int64_t><<<1, ALIGN_WARPS * 32, smem, stream>>>(
        static_cast<const int64_t *>(topk_ids), numel, num_experts, block_size, expert_map, map_mode, sorted_ids,
        sorted_capacity, expert_ids, expert_ids_capacity, num_tokens_post_pad, chunks, num_chunks, chunk_capacity, inv_pos, chunk_max);
  } else {
    return fail(LO_ERR_UNSUPPORTED, "moe_align: unsupported id dtype code %d", ids_dtype);
  }
  LO_LAUNCH_OK("align_kernel");
  return LO_OK;
}

int launch_chunks_from_blocks(const int32_t *expert_ids, const int32_t *num_tokens_post_pad, int block_size,
                              int64_t max_blocks, Chunk *chunks, int32_t *num_chunks, cudaStream_t stream) {
  const int per_block = block_size <= 128 ? 1 : block_size / 128;
  const int64_t n = max_blocks * per_block;
  const int blocks = (int)(ceil_div(n, 256) < 1 ? 1 : (ceil_div(n, 256) > 1024 ? 1024 : ceil_div(n, 256)));
  chunks_from_blocks_kernel<<<blocks, 256, 0, stream>>>(expert_ids, num_tokens_post_pad, block_size, max_blocks,
                                                       chunks, num_chunks);
  LO_LAUNCH_OK("chunks_from_blocks_kernel");
  return LO_OK;
}

}  // namespace lo

extern "C" int lo_topk_softmax(const void *gating, int gating_dtype, int64_t M, int E, int k, int renormalize,
                               float *topk_weights, void *topk_ids, int ids_dtype,
                               int32_t *token_expert_indices, void *stream) {
  using namespace lo;
  LO_REQUIRE(M >= 0, "topk_softmax: negative row count");
  if (M == 0) return LO_OK;
  LO_REQUIRE(gating && topk_weights && topk_ids, "topk_softmax: null pointer");
  LO_REQUIRE(E >= 1 && E <= 1024, "topk_softmax: num_experts %d outside [1,1024]", E);
  LO_REQUIRE(k >= 1 && k <= 32 && k <= E, "topk_softmax: top_k %d outside [1,min(32,E)]", k);
  LO_REQUIRE(ceil_div(M, 8) <= 0x7fffffffLL, "topk_softmax: too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (gating_dtype) {
    case LO_F32: return launch_topk_ids<float>(gating, M, E, k, renormalize, topk_weights, topk_ids, ids_dtype, token_expert_indices, st);
    case LO_F16: return launch_topk_ids<__half>(gating, M, E, k, renormalize, topk_weights, topk_ids, ids_dtype, token_expert_indices, st);
    case LO_BF16: return launch_topk_ids<__nv_bfloat16>(gating, M, E, k, renormalize, topk_weights, topk_ids, ids_dtype, token_expert_indices, st);
    default: return fail(LO_ERR_UNSUPPORTED, "topk_softmax: unsupported gating dtype code %d", gating_dtype);
  }
}

extern "C" int lo_moe_align_block_size(const void *topk_ids, int ids_dtype, int64_t numel, int num_experts,
                                       int block_size, const int32_t *expert_map, int map_mode,
                                       int32_t *sorted_ids, int64_t sorted_capacity, int32_t *expert_ids,
                                       int64_t expert_ids_capacity, int32_t *num_tokens_post_pad, void *stream) {
  return lo::launch_align(topk_ids, ids_dtype, numel, num_experts, block_size, expert_map, map_mode, sorted_ids,
                          sorted_capacity, expert_ids, expert_ids_capacity, num_tokens_post_pad, nullptr, nullptr,
                          0, nullptr, 128, static_cast<cudaStream_t>(stream));
}
