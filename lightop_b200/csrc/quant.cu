// Per-token-group INT8 quantisation (bf16 / fp16 / fp32 -> int8 + fp32 scale per group).
//
// Arithmetic (must stay bit-identical to the reference's torch model,
// test/moe_w8a8/benchmark_moe_int8.py:60-83):
//   amax  = max |x| over the group, clamped from below by eps rounded to x's type
//   scale = amax / 127                 (IEEE fp32 division)
//   q     = trunc(clamp(x / scale, -128, 127))   (IEEE fp32 division, then round toward zero)
// Memory-bound streaming kernel: LANES lanes own one group, each lane moves 16
// bytes of 2-byte input (or 32 bytes of fp32) and stores 8 int8 in one 8-byte store.
#include "common.h"

namespace lo {
namespace {

template <typename T> struct Load8;
template <> struct Load8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&v)[8]) {
    uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
template <> struct Load8<__half> {
  static __device__ __forceinline__ void load(const __half *p, float (&v)[8]) {
    uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};
template <> struct Load8<float> {
  static __device__ __forceinline__ void load(const float *p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4 *>(p);
    float4 b = *reinterpret_cast<const float4 *>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};

// LANES lanes x 8 elements = one group.
template <typename T, int LANES>
__global__ void __launch_bounds__(256) group_quant_kernel(const T *__restrict__ x, int8_t *__restrict__ q,
                                                          float *__restrict__ s, int64_t num_groups,
                                                          float eps_t) {
  const int64_t gthread = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t group = gthread / LANES;
  const int lane_in_group = (int)(gthread % LANES);
  const bool active = group < num_groups;
  float v[8];
  float amax = 0.f;
  if (active) {
    Load8<T>::load(x + group * (LANES * 8) + lane_in_group * 8, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
#pragma unroll
  for (int off = LANES / 2; off > 0; off >>= 1)
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if (!active) return;
  amax = fmaxf(amax, eps_t);
  const float scale = __fdiv_rn(amax, 127.0f);
  uint32_t packed[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float r = __fdiv_rn(v[i], scale);
    r = fminf(fmaxf(r, -128.0f), 127.0f);
    const int qi = __float2int_rz(r);
    packed[i >> 2] |= (uint32_t)(qi & 0xff) << (8 * (i & 3));
  }
  *reinterpret_cast<uint2 *>(q + group * (LANES * 8) + lane_in_group * 8) = make_uint2(packed[0], packed[1]);
  if (lane_in_group == 0) s[group] = scale;
}

// bf16 rows [M, H], group 128: quantise once, store to each of the token's sorted positions.
__global__ void __launch_bounds__(256) group_quant_scatter_kernel(const __nv_bfloat16 *__restrict__ x, int64_t M,
                                                                  int64_t groups_per_row, int topk,
                                                                  const int32_t *__restrict__ inv_pos, float eps_t,
                                                                  int8_t *__restrict__ q_sorted,
                                                                  float *__restrict__ s_sorted) {
  const int64_t gthread = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t group = gthread / 16;
  const int lane_in_group = (int)(gthread % 16);
  const bool active = group < M * groups_per_row;
  float v[8];
  float amax = 0.f;
  if (active) {
    Load8<__nv_bfloat16>::load(x + group * 128 + lane_in_group * 8, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if (!active) return;
  amax = fmaxf(amax, eps_t);
  const float scale = __fdiv_rn(amax, 127.0f);
  uint32_t packed[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float r = __fdiv_rn(v[i], scale);
    r = fminf(fmaxf(r, -128.0f), 127.0f);
    packed[i >> 2] |= (uint32_t)(__float2int_rz(r) & 0xff) << (8 * (i & 3));
  }
  const int64_t token = group / groups_per_row;
  const int64_t gi = group % groups_per_row;
  for (int j = 0; j < topk; ++j) {
    const int32_t pos = inv_pos[token * topk + j];
    if (pos < 0) continue;
    *reinterpret_cast<uint2 *>(q_sorted + ((int64_t)pos * groups_per_row + gi) * 128 + lane_in_group * 8) =
        make_uint2(packed[0], packed[1]);
    if (lane_in_group == 0) s_sorted[(int64_t)pos * groups_per_row + gi] = scale;
  }
}

template <typename T>
int launch_typed(const void *x, int64_t num_groups, int group_size, float eps_t, int8_t *q, float *s,
                 cudaStream_t stream) {
  const int lanes = group_size / 8;
  const int threads = 256;
  const int64_t total_threads = num_groups * lanes;
  const int64_t blocks = ceil_div(total_threads, threads);
  if (blocks > 0x7fffffffLL) return fail(LO_ERR_INVALID_ARGUMENT, "group quant: too many groups");
  const T *xp = static_cast<const T *>(x);
  switch (lanes) {
    case 8: group_quant_kernel<T, 8><<<(unsigned)blocks, threads, 0, stream>>>(xp, q, s, num_groups, eps_t); break;
    case 16: group_quant_kernel<T, 16><<<(unsigned)blocks, threads, 0, stream>>>(xp, q, s, num_groups, eps_t); break;
    case 32: group_quant_kernel<T, 32><<<(unsigned)blocks, threads, 0, stream>>>(xp, q, s, num_groups, eps_t); break;
    default: return fail(LO_ERR_UNSUPPORTED, "group quant: group_size %d not in {64,128,256}", group_size);
  }
  LO_LAUNCH_OK("group_quant_kernel");
  return LO_OK;
}

}  // namespace

// eps rounded to the element type of x, the way a torch clamp(min=eps) on a tensor of
// that type sees it.
float round_eps_to_dtype(float eps, int dtype) {
  if (dtype == LO_BF16) return __bfloat162float(__float2bfloat16_rn(eps));
  if (dtype == LO_F16) return __half2float(__float2half_rn(eps));
  return eps;
}

int launch_group_quant_scatter(const void *x, int64_t M, int64_t H, int topk, const int32_t *inv_pos, float eps,
                               int8_t *q_sorted, float *s_sorted, cudaStream_t stream) {
  if (M == 0) return LO_OK;
  LO_REQUIRE(H % 128 == 0, "group quant: hidden size must be a multiple of 128");
  const int64_t total_threads = M * (H / 128) * 16;
  const int64_t blocks = ceil_div(total_threads, 256);
  LO_REQUIRE(blocks <= 0x7fffffffLL, "group quant: too many groups");
  group_quant_scatter_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x), M, H / 128, topk,
                                                                   inv_pos, round_eps_to_dtype(eps, LO_BF16), q_sorted,
                                                                   s_sorted);
  LO_LAUNCH_OK("group_quant_scatter_kernel");
  return LO_OK;
}

}  // namespace lo

extern "C" int lo_group_quant_int8(const void *x, int x_dtype, int64_t num_groups, int group_size,
                                   float eps, int8_t *q, float *s, void *stream) {
  using namespace lo;
  LO_REQUIRE(num_groups >= 0, "group quant: negative group count");
  if (num_groups == 0) return LO_OK;
  LO_REQUIRE(x && q && s, "group quant: null pointer");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
             "group quant: x must be 16-byte and q 8-byte aligned");
  const float eps_t = round_eps_to_dtype(eps, x_dtype);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case LO_BF16: return launch_typed<__nv_bfloat16>(x, num_groups, group_size, eps_t, q, s, st);
    case LO_F16: return launch_typed<__half>(x, num_groups, group_size, eps_t, q, s, st);
    case LO_F32: return launch_typed<float>(x, num_groups, group_size, eps_t, q, s, st);
    default: return fail(LO_ERR_UNSUPPORTED, "group quant: unsupported input dtype code %d", x_dtype);
  }
}
