// Grouped, bias-corrected sigmoid gate (the DeepSeek-V3 router) and the top-k id post-processing.
//
// moe_fused_gate, per token (one warp per token, experts strided over the lanes):
//   p[e]      = sigmoid(x[e])                          (fp32)
//   s[e]      = p[e] + bias[e]                         (selection score)
//   group g   = experts [g*S, (g+1)*S), S = E / groups; group score = sum of its two largest s
//   keep the topk_group best groups (ties: lower group), mask the others out
//   pick the k_routed = topk - shared best s among the kept experts (ties: lower expert id),
//   in descending order
//   weight    = p[chosen] / sum(p[chosen]) * (routed_scaling_factor if applied on output)
//   shared experts (fused in as extra slots): id = E + j, weight = (1 / routed_scaling_factor) * same factor
// Selection runs on registers; the group phase goes through a per-warp row of s in shared memory,
// lane g scanning group g, so any group size works.
#include "common.h"

namespace lo {
namespace {

constexpr int GATE_WARPS = 4;

__device__ __forceinline__ float load_as_float(const void *p, int dtype, int64_t i) {
  if (dtype == LO_F32) return static_cast<const float *>(p)[i];
  if (dtype == LO_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
  return __half2float(static_cast<const __half *>(p)[i]);
}

template <int VPL, typename IdT>
__global__ void __launch_bounds__(GATE_WARPS * 32) fused_gate_kernel(
    const void *__restrict__ x, int x_dtype, const void *__restrict__ bias, int bias_dtype, int64_t M, int E,
    int groups, int topk_group, int topk, int n_shared, float scaling, int scale_on_output,
    float *__restrict__ weights, IdT *__restrict__ ids) {
  extern __shared__ float gate_smem[];              // [GATE_WARPS][2][E]: selection scores, probabilities
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t row = (int64_t)blockIdx.x * GATE_WARPS + warp;
  if (row >= M) return;
  float *s_row = gate_smem + (size_t)warp * 2 * E;
  float *p_row = s_row + E;
  const int S = E / groups;
  const int k_routed = topk - n_shared;

  float s[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int e = lane + 32 * i;
    s[i] = -INFINITY;
    if (e < E) {
      const float v = load_as_float(x, x_dtype, row * E + e);
      const float p = 1.0f / (1.0f + expf(-v));
      s[i] = p + load_as_float(bias, bias_dtype, e);
      s_row[e] = s[i];
      p_row[e] = p;
    }
  }
  __syncwarp();

  if (groups > 1) {
    // lane g: sum of the two largest scores of group g
    float gscore = -INFINITY;
    if (lane < groups) {
      float m1 = -INFINITY, m2 = -INFINITY;
      for (int j = 0; j < S; ++j) {
        const float v = s_row[lane * S + j];
        if (v > m1) { m2 = m1; m1 = v; }
        else if (v > m2) { m2 = v; }
      }
      gscore = m1 + m2;
    }
    uint32_t keep = 0u;           // bit g: group g survives
    for (int r = 0; r < topk_group; ++r) {
      float best = gscore;
      int best_g = lane;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int og = __shfl_xor_sync(0xffffffffu, best_g, off);
        if (ob > best || (ob == best && og < best_g)) { best = ob; best_g = og; }
      }
      keep |= 1u << best_g;
      if (lane == best_g) gscore = -INFINITY;
    }
    // lanes >= groups hold -inf and a lane index >= groups; a winner among them would mean fewer than
    // topk_group finite groups, which the argument checks exclude for finite inputs
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int e = lane + 32 * i;
      if (e < E && !((keep >> (e / S)) & 1u)) s[i] = -INFINITY;
    }
  }

  float my_p = 0.f;
  int my_id = 0;
  float p_sum = 0.f;
  for (int r = 0; r < k_routed; ++r) {
    float best = s[0];
    int best_e = lane;
#pragma unroll
    for (int i = 1; i < VPL; ++i) {
      if (s[i] > best) { best = s[i]; best_e = lane + 32 * i; }      // strict: the lower id stays on ties
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    const float p = p_row[best_e < E ? best_e : 0];
    p_sum += p;
    if (lane == r) { my_p = p; my_id = best_e; }
    if ((best_e & 31) == lane) {
      const int slot = best_e >> 5;
#pragma unroll
      for (int i = 0; i < VPL; ++i)
        if (i == slot) s[i] = -INFINITY;
    }
  }
  if (lane >= k_routed && lane < topk) {
    my_id = E + (lane - k_routed);
    my_p = p_sum / (scaling > 0.f ? scaling : 1.0f);
  }
  if (lane < topk) {
    const float route_scale = (scale_on_output && scaling > 0.f) ? scaling : 1.0f;
    weights[row * topk + lane] = (my_p / p_sum) * route_scale;
    ids[row * topk + lane] = (IdT)my_id;
  }
}

template <typename IdT>
int launch_gate(const void *x, int x_dtype, const void *bias, int bias_dtype, int64_t M, int E, int groups,
                int topk_group, int topk, int n_shared, float scaling, int on_output, float *w, void *ids,
                cudaStream_t st) {
  const int64_t blocks = ceil_div(M, GATE_WARPS);
  const size_t smem = (size_t)GATE_WARPS * 2 * E * sizeof(float);
  IdT *idp = static_cast<IdT *>(ids);
  const int vpl = (int)ceil_div(E, 32);
#define LO_GATE_CASE(V)                                                                                         \
  fused_gate_kernel<V, IdT><<<(unsigned)blocks, GATE_WARPS * 32, smem, st>>>(x, x_dtype, bias, bias_dtype, M, E, groups, \
                                                                             topk_group, topk, n_shared, scaling,  \
                                                                             on_output, w, idp)
  if (vpl <= 4) LO_GATE_CASE(4);
  else if (vpl <= 8) LO_GATE_CASE(8);
  else if (vpl <= 16) LO_GATE_CASE(16);
  else LO_GATE_CASE(32);
#undef LO_GATE_CASE
  LO_LAUNCH_OK("fused_gate_kernel");
  return LO_OK;
}

// topk_ids_postprocess: ids of tokens at or beyond *num_token_non_padded become -1; the others go through
// the logical -> physical expert map (ids outside the map become -1).  Both steps are optional.
template <typename IdT>
__global__ void ids_postprocess_kernel(IdT *__restrict__ ids, int64_t total, int64_t topk, const void *__restrict__ map,
                                       int map_dtype, int64_t map_size, const void *__restrict__ num_valid,
                                       int num_valid_dtype) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  if (num_valid) {
    const int64_t nv = num_valid_dtype == LO_I64 ? *static_cast<const int64_t *>(num_valid)
                                                 : (int64_t) * static_cast<const int32_t *>(num_valid);
    if (i / topk >= nv) {
      ids[i] = (IdT)-1;
      return;
    }
  }
  if (!map) return;
  const int64_t e = (int64_t)ids[i];
  int64_t phys = -1;
  if (e >= 0 && e < map_size)
    phys = map_dtype == LO_I64 ? static_cast<const int64_t *>(map)[e] : (int64_t) static_cast<const int32_t *>(map)[e];
  ids[i] = (IdT)phys;
}

}  // namespace
}  // namespace lo

extern "C" int lo_moe_fused_gate(const void *x, int x_dtype, const void *bias, int bias_dtype, int64_t M, int E,
                                 int num_expert_group, int topk_group, int topk, int n_share_experts_fusion,
                                 float routed_scaling_factor, int apply_routed_scaling_factor_on_output,
                                 float *topk_weights, void *topk_ids, int ids_dtype, void *stream) {
  using namespace lo;
  LO_REQUIRE(M >= 0 && E >= 1 && E <= 1024, "moe_fused_gate: expert count %d out of range (1..1024)", E);
  LO_REQUIRE(x_dtype == LO_F32 || x_dtype == LO_F16 || x_dtype == LO_BF16, "moe_fused_gate: unsupported input dtype code %d", x_dtype);
  LO_REQUIRE(bias_dtype == LO_F32 || bias_dtype == LO_F16 || bias_dtype == LO_BF16, "moe_fused_gate: unsupported bias dtype code %d", bias_dtype);
  // the reference's own argument rules (csrc/kernels/moe_gate/moe_fused_gate.cu:1352-1368)
  LO_REQUIRE(num_expert_group > 0 && num_expert_group <= E && E % num_expert_group == 0,
             "moe_fused_gate: invalid num_expert_group=%d for experts=%d", num_expert_group, E);
  LO_REQUIRE(num_expert_group <= 32, "moe_fused_gate: at most 32 expert groups");
  LO_REQUIRE(topk_group > 0 && topk_group <= num_expert_group,
             "moe_fused_gate: topk_group must be in [1, num_expert_group], got %d with num_expert_group=%d", topk_group, num_expert_group);
  LO_REQUIRE(topk > 0 && topk <= 32 && n_share_experts_fusion >= 0 && n_share_experts_fusion < topk &&
                 topk - n_share_experts_fusion <= (E / num_expert_group) * topk_group,
             "moe_fused_gate: invalid topk/shared-expert configuration: topk=%d, shared=%d, experts=%d, groups=%d, topk_group=%d",
             topk, n_share_experts_fusion, E, num_expert_group, topk_group);
  LO_REQUIRE(routed_scaling_factor == routed_scaling_factor && routed_scaling_factor - routed_scaling_factor == 0.f,
             "moe_fused_gate: routed_scaling_factor must be finite");
  if (M == 0) return LO_OK;
  LO_REQUIRE(x && bias && topk_weights && topk_ids, "moe_fused_gate: null pointer");
  LO_REQUIRE(M <= 0x7fffffffLL * GATE_WARPS, "moe_fused_gate: too many tokens");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_dtype == LO_I64)
    return launch_gate<int64_t>(x, x_dtype, bias, bias_dtype, M, E, num_expert_group, topk_group, topk, n_share_experts_fusion,
                                routed_scaling_factor, apply_routed_scaling_factor_on_output, topk_weights, topk_ids, st);
  LO_REQUIRE(ids_dtype == LO_I32, "moe_fused_gate: indices must be int32 or int64");
  return launch_gate<int32_t>(x, x_dtype, bias, bias_dtype, M, E, num_expert_group, topk_group, topk, n_share_experts_fusion,
                              routed_scaling_factor, apply_routed_scaling_factor_on_output, topk_weights, topk_ids, st);
}

extern "C" int lo_topk_ids_postprocess(void *topk_ids, int ids_dtype, int64_t M, int64_t topk,
                                       const void *logical_to_physical_map, int map_dtype, int64_t map_size,
                                       const void *num_token_non_padded, int num_token_dtype, void *stream) {
  using namespace lo;
  LO_REQUIRE(M >= 0 && topk >= 1, "topk_ids_postprocess: bad shape");
  const int64_t total = M * topk;
  if (total == 0) return LO_OK;
  LO_REQUIRE(topk_ids != nullptr, "topk_ids_postprocess: null ids");
  LO_REQUIRE(ids_dtype == LO_I32 || ids_dtype == LO_I64, "topk_ids_postprocess expects int32 or int64 tensor");
  LO_REQUIRE(!logical_to_physical_map || map_dtype == LO_I32 || map_dtype == LO_I64,
             "topk_ids_postprocess: the map must be int32 or int64");
  LO_REQUIRE(!num_token_non_padded || num_token_dtype == LO_I32 || num_token_dtype == LO_I64,
             "topk_ids_postprocess: num_token_non_padded must be int32 or int64");
  const int64_t blocks = ceil_div(total, 256);
  LO_REQUIRE(blocks <= 0x7fffffffLL, "topk_ids_postprocess: too many ids");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_dtype == LO_I64)
    ids_postprocess_kernel<int64_t><<<(unsigned)blocks, 256, 0, st>>>(static_cast<int64_t *>(topk_ids), total, topk,
                                                                     logical_to_physical_map, map_dtype, map_size,
                                                                     num_token_non_padded, num_token_dtype);
  else
    ids_postprocess_kernel<int32_t><<<(unsigned)blocks, 256, 0, st>>>(static_cast<int32_t *>(topk_ids), total, topk,
                                                                     logical_to_physical_map, map_dtype, map_size,
                                                                     num_token_non_padded, num_token_dtype);
  LO_LAUNCH_OK("ids_postprocess_kernel");
  return LO_OK;
}
