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
// The kernel takes the score function (sigmoid or sqrt(softplus)), whether to renormalise, the epsilon of the
// normalisation, the output factor and the shared-expert divisor as parameters, which also covers the
// reference's ungrouped variants (Kimi-K2 gate, sqrt-softplus gate).
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
    const void *__restrict__ x, int x_dtype, const void *__restrict__ bias, int bias_dtype, int64_t bias_row_stride,
    int64_t M, int E, int groups, int topk_group, int topk, int n_shared, int score_fn, int renormalize, float norm_eps,
    float out_scale, float shared_div, const void *__restrict__ num_valid, int num_valid_dtype, int padding_id,
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
      // unbiased score of the expert: sigmoid(v), or sqrt(softplus(v)) (the second form takes softplus(v) = v
      // beyond 20, where the two agree to fp32 precision, and so never overflows)
      float p;
      if (score_fn == LO_GATE_SIGMOID) p = 1.0f / (1.0f + expf(-v));
      else p = sqrtf(score_fn == LO_GATE_SQRT_SOFTPLUS_SAFE && v > 20.0f ? v : log1pf(expf(v)));
      s[i] = p + load_as_float(bias, bias_dtype, row * bias_row_stride + e);
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
    my_p = p_sum / shared_div;
  }
  if (lane < topk) {
    float denom = renormalize ? p_sum + norm_eps : 1.0f;
    // csrc/kernels/moe_gate/moe_fused_gate_sqrtsoftplus.cu:202: a row whose routed scores are all zero is not normalised
    if (score_fn != LO_GATE_SIGMOID && !(p_sum > 0.f)) denom = 1.0f;
    // rows at or beyond the device-side count of real tokens: weight 0 and the caller's padding id (same file, :205-212)
    bool padded = false;
    if (num_valid)
      padded = row >= (num_valid_dtype == LO_I64 ? *static_cast<const int64_t *>(num_valid)
                                                 : (int64_t) * static_cast<const int32_t *>(num_valid));
    weights[row * topk + lane] = padded ? 0.f : (my_p / denom) * out_scale;
    ids[row * topk + lane] = padded ? (IdT)padding_id : (IdT)my_id;
  }
}

template <typename IdT>
int launch_gate(const void *x, int x_dtype, const void *bias, int bias_dtype, int64_t bias_row_stride, int64_t M, int E, int groups,
                int topk_group, int topk, int n_shared, int score_fn, int renormalize, float norm_eps, float out_scale,
                float shared_div, const void *num_valid, int num_valid_dtype, int padding_id, float *w, void *ids,
                cudaStream_t st) {
  const int64_t blocks = ceil_div(M, GATE_WARPS);
  const size_t smem = (size_t)GATE_WARPS * 2 * E * sizeof(float);
  IdT *idp = static_cast<IdT *>(ids);
  const int vpl = (int)ceil_div(E, 32);
#define LO_GATE_CASE(V)                                                                                         \
  fused_gate_kernel<V, IdT><<<(unsigned)blocks, GATE_WARPS * 32, smem, st>>>(x, x_dtype, bias, bias_dtype, bias_row_stride, M, E, groups, \
                                                                             topk_group, topk, n_shared, score_fn, \
                                                                             renormalize, norm_eps, out_scale,     \
                                                                             shared_div, num_valid, num_valid_dtype,\
                                                                             padding_id, w, idp)
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

extern "C" int lo_moe_gate_topk(const void *x, int x_dtype, const void *bias, int bias_dtype, int64_t bias_row_stride,
                                int64_t M, int E,
                                int num_expert_group, int topk_group, int topk, int n_shared, int score_fn,
                                int renormalize, float norm_eps, float out_scale, float shared_div,
                                const void *num_token_non_padded, int num_token_dtype, int padding_id,
                                float *topk_weights, void *topk_ids, int ids_dtype, void *stream) {
  using namespace lo;
  LO_REQUIRE(M >= 0 && E >= 1 && E <= 1024, "moe gate: expert count %d out of range (1..1024)", E);
  LO_REQUIRE(x_dtype == LO_F32 || x_dtype == LO_F16 || x_dtype == LO_BF16, "moe gate: unsupported input dtype code %d", x_dtype);
  LO_REQUIRE(bias_dtype == LO_F32 || bias_dtype == LO_F16 || bias_dtype == LO_BF16, "moe gate: unsupported bias dtype code %d", bias_dtype);
  LO_REQUIRE(score_fn == LO_GATE_SIGMOID || score_fn == LO_GATE_SQRT_SOFTPLUS || score_fn == LO_GATE_SQRT_SOFTPLUS_SAFE,
             "moe gate: unknown score function %d", score_fn);
  // the reference's own argument rules (csrc/kernels/moe_gate/moe_fused_gate.cu:1352-1368)
  LO_REQUIRE(num_expert_group > 0 && num_expert_group <= E && E % num_expert_group == 0,
             "moe gate: invalid num_expert_group=%d for experts=%d", num_expert_group, E);
  LO_REQUIRE(num_expert_group <= 32, "moe gate: at most 32 expert groups");
  LO_REQUIRE(topk_group > 0 && topk_group <= num_expert_group,
             "moe gate: topk_group must be in [1, num_expert_group], got %d with num_expert_group=%d", topk_group, num_expert_group);
  LO_REQUIRE(topk > 0 && topk <= 32 && n_shared >= 0 && n_shared < topk && topk - n_shared <= (E / num_expert_group) * topk_group,
             "moe gate: invalid topk/shared-expert configuration: topk=%d, shared=%d, experts=%d, groups=%d, topk_group=%d",
             topk, n_shared, E, num_expert_group, topk_group);
  LO_REQUIRE(out_scale - out_scale == 0.f && shared_div - shared_div == 0.f && shared_div != 0.f,
             "moe gate: the scaling factors must be finite and the shared-expert divisor non-zero");
  LO_REQUIRE(bias_row_stride == 0 || bias_row_stride >= E, "moe gate: a per-token bias needs a row stride of at least %d", E);
  LO_REQUIRE(!num_token_non_padded || num_token_dtype == LO_I32 || num_token_dtype == LO_I64,
             "moe gate: num_token_non_padded must be int32 or int64");
  if (M == 0) return LO_OK;
  LO_REQUIRE(x && bias && topk_weights && topk_ids, "moe gate: null pointer");
  LO_REQUIRE(M <= 0x7fffffffLL * GATE_WARPS, "moe gate: too many tokens");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_dtype == LO_I64)
    return launch_gate<int64_t>(x, x_dtype, bias, bias_dtype, bias_row_stride, M, E, num_expert_group, topk_group, topk, n_shared, score_fn,
                                renormalize, norm_eps, out_scale, shared_div, num_token_non_padded, num_token_dtype, padding_id,
                                topk_weights, topk_ids, st);
  LO_REQUIRE(ids_dtype == LO_I32, "moe gate: indices must be int32 or int64");
  return launch_gate<int32_t>(x, x_dtype, bias, bias_dtype, bias_row_stride, M, E, num_expert_group, topk_group, topk, n_shared, score_fn,
                              renormalize, norm_eps, out_scale, shared_div, num_token_non_padded, num_token_dtype, padding_id,
                                topk_weights, topk_ids, st);
}

extern "C" int lo_moe_fused_gate(const void *x, int x_dtype, const void *bias, int bias_dtype, int64_t M, int E,
                                 int num_expert_group, int topk_group, int topk, int n_share_experts_fusion,
                                 float routed_scaling_factor, int apply_routed_scaling_factor_on_output,
                                 float *topk_weights, void *topk_ids, int ids_dtype, void *stream) {
  using namespace lo;
  LO_REQUIRE(routed_scaling_factor == routed_scaling_factor && routed_scaling_factor - routed_scaling_factor == 0.f,
             "moe_fused_gate: routed_scaling_factor must be finite");
  // csrc/kernels/moe_gate/moe_fused_gate.cu:296-311: a factor <= 0 counts as 1, for the output and for the shared experts
  const float factor = routed_scaling_factor > 0.f ? routed_scaling_factor : 1.0f;
  return lo_moe_gate_topk(x, x_dtype, bias, bias_dtype, 0, M, E, num_expert_group, topk_group, topk, n_share_experts_fusion,
                          LO_GATE_SIGMOID, 1, 0.f, apply_routed_scaling_factor_on_output ? factor : 1.0f, factor,
                          nullptr, 0, 0, topk_weights, topk_ids, ids_dtype, stream);
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
