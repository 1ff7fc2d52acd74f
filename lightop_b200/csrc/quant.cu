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
  if (!active) return;          // (an exited block counts as released for the dependent launch)
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
  // everything above reads the caller's activations only; the positions come from the align kernel before this one
  dependency_wait();
  dependency_release();
  for (int j = 0; j < topk; ++j) {
    const int32_t pos = inv_pos[token * topk + j];
    if (pos < 0) continue;
    *reinterpret_cast<uint2 *>(q_sorted + ((int64_t)pos * groups_per_row + gi) * 128 + lane_in_group * 8) =
        make_uint2(packed[0], packed[1]);
    if (lane_in_group == 0) s_sorted[(int64_t)pos * groups_per_row + gi] = scale;
  }
}

// ---------------------------------------------------------------------------
// Per-token (whole-row) INT8 quantisation, the activation format of the per-channel W8A8 mode.
//
// Arithmetic of the reference's kernel (python/lightop/_lmslim_native/layers/gemm/int8_utils.py:21-44):
//   absmax = max(max |x|, 1e-10)       (fp32)
//   scale  = absmax / 127              (IEEE fp32 division)
//   q      = rint(x * (127 / absmax))  (one fp32 division per row, fp32 product, round half to even)
// One CTA per row: pass 1 takes the maximum, pass 2 re-reads the row (it is still in L1/L2) and
// stores 8 int8 per thread and step.  With inv_pos the int8 row and its scale are written to every
// sorted position of the token instead of to row `token` (same layout trick as the group kernel).
// ---------------------------------------------------------------------------
constexpr int TOKEN_QUANT_THREADS = 256;

__device__ __forceinline__ float block_max_256(float v, float *red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[lane & 7];
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, off));
  __syncthreads();   // red may be reused by the caller
  return r;
}

__device__ __forceinline__ uint2 quant8_rn(const float (&v)[8], float inv) {
  uint32_t packed[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float r = __fmul_rn(v[i], inv);
    r = fminf(fmaxf(r, -128.0f), 127.0f);
    packed[i >> 2] |= (uint32_t)(__float2int_rn(r) & 0xff) << (8 * (i & 3));
  }
  return make_uint2(packed[0], packed[1]);
}

template <typename T>
__global__ void __launch_bounds__(TOKEN_QUANT_THREADS) token_quant_kernel(const T *__restrict__ x, int64_t K, int topk,
                                                                          const int32_t *__restrict__ inv_pos,
                                                                          int8_t *__restrict__ q, float *__restrict__ s) {
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  const T *xr = x + row * K;
  // rows of a length that is not a multiple of 8 are not 16-byte aligned: they take the scalar loops only
  const int64_t vecs = (K & 7) == 0 ? K / 8 : 0;
  float amax = 0.f;
  for (int64_t i = threadIdx.x; i < vecs; i += TOKEN_QUANT_THREADS) {
    float v[8];
    Load8<T>::load(xr + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  }
  for (int64_t i = vecs * 8 + threadIdx.x; i < K; i += TOKEN_QUANT_THREADS) amax = fmaxf(amax, fabsf((float)xr[i]));
  amax = fmaxf(block_max_256(amax, red), 1e-10f);
  const float scale = __fdiv_rn(amax, 127.0f);
  const float inv = __fdiv_rn(127.0f, amax);
  if (inv_pos == nullptr) {
    for (int64_t i = threadIdx.x; i < vecs; i += TOKEN_QUANT_THREADS) {
      float v[8];
      Load8<T>::load(xr + i * 8, v);
      *reinterpret_cast<uint2 *>(q + row * K + i * 8) = quant8_rn(v, inv);
    }
    for (int64_t i = vecs * 8 + threadIdx.x; i < K; i += TOKEN_QUANT_THREADS) {
      const float r = fminf(fmaxf(__fmul_rn((float)xr[i], inv), -128.0f), 127.0f);
      q[row * K + i] = (int8_t)__float2int_rn(r);
    }
    if (threadIdx.x == 0) s[row] = scale;
    return;
  }
  for (int64_t i = threadIdx.x; i < vecs; i += TOKEN_QUANT_THREADS) {
    float v[8];
    Load8<T>::load(xr + i * 8, v);
    const uint2 pk = quant8_rn(v, inv);
    for (int j = 0; j < topk; ++j) {
      const int32_t pos = inv_pos[row * topk + j];
      if (pos >= 0) *reinterpret_cast<uint2 *>(q + (int64_t)pos * K + i * 8) = pk;
    }
  }
  if (threadIdx.x < topk) {
    const int32_t pos = inv_pos[row * topk + threadIdx.x];
    if (pos >= 0) s[pos] = scale;
  }
}

// ---------------------------------------------------------------------------
// SiLU(gate) * up followed by per-token INT8 quantisation, one CTA per row of a bf16 [rows, 2*d]
// matrix (gate columns first).  Semantics of the reference's fused kernel
// (csrc/kernels/gated_activation/fuse_silu_mul_quant.cu:90-131) with exact fp32 expf / division in
// the SiLU: act = bf16(bf16(silu(gate)) * up); scale = max|act| / 127; q = rint(act * (127 / max)),
// saturated; a row of zeros gets scale 0 and q 0.  Rows whose entry in row_ids is a padding
// sentinel (< 0 or >= numel_valid) are skipped.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(TOKEN_QUANT_THREADS) silu_mul_token_quant_kernel(
    const __nv_bfloat16 *__restrict__ in, int64_t d, const int32_t *__restrict__ row_ids, int64_t numel_valid,
    const int32_t *__restrict__ num_rows_dev, int64_t group_rows, const int32_t *__restrict__ group_counts,
    int8_t *__restrict__ q, float *__restrict__ s) {
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  if (num_rows_dev && row >= *num_rows_dev) return;
  // masked layout [groups, group_rows, 2d]: only the first group_counts[g] rows of a group exist
  if (group_counts && row % group_rows >= group_counts[row / group_rows]) return;
  if (row_ids) {
    const int32_t id = row_ids[row];
    if (id < 0 || id >= numel_valid) return;
  }
  const __nv_bfloat16 *g = in + row * 2 * d;
  const __nv_bfloat16 *u = g + d;
  const int64_t vecs = d / 8;
  float amax = 0.f;
  if (vecs <= 2 * TOKEN_QUANT_THREADS) {
    // rows of up to 4096 channels: the activations stay in registers between the maximum and the
    // quantisation (one read of the row, one evaluation of the SiLU)
    float av[2][8];
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      const int64_t i = threadIdx.x + (int64_t)v * TOKEN_QUANT_THREADS;
      if (i < vecs) {
        float gv[8], uv[8];
        Load8<__nv_bfloat16>::load(g + i * 8, gv);
        Load8<__nv_bfloat16>::load(u + i * 8, uv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float sl = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(gv[j], 1.0f + expf(-gv[j]))));
          av[v][j] = __bfloat162float(__float2bfloat16_rn(sl * uv[j]));
          amax = fmaxf(amax, fabsf(av[v][j]));
        }
      }
    }
    amax = block_max_256(amax, red);
    const float inv = amax == 0.f ? 0.f : __fdiv_rn(127.0f, amax);
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      const int64_t i = threadIdx.x + (int64_t)v * TOKEN_QUANT_THREADS;
      if (i < vecs) *reinterpret_cast<uint2 *>(q + row * d + i * 8) = quant8_rn(av[v], inv);
    }
    if (threadIdx.x == 0) s[row] = __fdiv_rn(amax, 127.0f);
    return;
  }
  for (int64_t i = threadIdx.x; i < vecs; i += TOKEN_QUANT_THREADS) {
    float gv[8], uv[8];
    Load8<__nv_bfloat16>::load(g + i * 8, gv);
    Load8<__nv_bfloat16>::load(u + i * 8, uv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sl = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(gv[j], 1.0f + expf(-gv[j]))));
      const float a = __bfloat162float(__float2bfloat16_rn(sl * uv[j]));
      amax = fmaxf(amax, fabsf(a));
    }
  }
  amax = block_max_256(amax, red);
  const float inv = amax == 0.f ? 0.f : __fdiv_rn(127.0f, amax);
  for (int64_t i = threadIdx.x; i < vecs; i += TOKEN_QUANT_THREADS) {
    float gv[8], uv[8], av[8];
    Load8<__nv_bfloat16>::load(g + i * 8, gv);
    Load8<__nv_bfloat16>::load(u + i * 8, uv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sl = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(gv[j], 1.0f + expf(-gv[j]))));
      av[j] = __bfloat162float(__float2bfloat16_rn(sl * uv[j]));
    }
    *reinterpret_cast<uint2 *>(q + row * d + i * 8) = quant8_rn(av, inv);
  }
  if (threadIdx.x == 0) s[row] = __fdiv_rn(amax, 127.0f);
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
  LO_CUDA_OK(launch_dependent(group_quant_scatter_kernel, dim3((unsigned)blocks), dim3(256), 0, stream,
                              static_cast<const __nv_bfloat16 *>(x), M, H / 128, topk, inv_pos,
                              round_eps_to_dtype(eps, LO_BF16), q_sorted, s_sorted));
  return LO_OK;
}

int launch_token_quant(const void *x, int x_dtype, int64_t M, int64_t K, int topk, const int32_t *inv_pos, int8_t *q,
                       float *s, cudaStream_t stream) {
  if (M == 0) return LO_OK;
  LO_REQUIRE(K >= 1, "per-token quant: empty rows");
  LO_REQUIRE(inv_pos == nullptr || K % 8 == 0, "per-token quant: the sorted layout needs a row length that is a multiple of 8");
  LO_REQUIRE(M <= 0x7fffffffLL, "per-token quant: too many rows");
  LO_REQUIRE(inv_pos == nullptr || (topk >= 1 && topk <= TOKEN_QUANT_THREADS), "per-token quant: bad top-k");
  const unsigned blocks = (unsigned)M;
  switch (x_dtype) {
    case LO_BF16:
      token_quant_kernel<__nv_bfloat16><<<blocks, TOKEN_QUANT_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x), K, topk, inv_pos, q, s);
      break;
    case LO_F16:
      token_quant_kernel<__half><<<blocks, TOKEN_QUANT_THREADS, 0, stream>>>(static_cast<const __half *>(x), K, topk, inv_pos, q, s);
      break;
    case LO_F32:
      token_quant_kernel<float><<<blocks, TOKEN_QUANT_THREADS, 0, stream>>>(static_cast<const float *>(x), K, topk, inv_pos, q, s);
      break;
    default: return fail(LO_ERR_UNSUPPORTED, "per-token quant: unsupported input dtype code %d", x_dtype);
  }
  LO_LAUNCH_OK("token_quant_kernel");
  return LO_OK;
}

int launch_silu_mul_token_quant(const void *in, int64_t rows, int64_t d, const int32_t *row_ids, int64_t numel_valid,
                                const int32_t *num_rows_dev, int8_t *q, float *s, cudaStream_t stream,
                                int64_t group_rows, const int32_t *group_counts) {
  if (rows == 0) return LO_OK;
  LO_REQUIRE(d >= 8 && d % 8 == 0, "silu-mul quant: width %lld must be a multiple of 8", (long long)d);
  LO_REQUIRE(rows <= 0x7fffffffLL, "silu-mul quant: too many rows");
  silu_mul_token_quant_kernel<<<(unsigned)rows, TOKEN_QUANT_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16 *>(in), d, row_ids, numel_valid, num_rows_dev, group_rows > 0 ? group_rows : 1,
      group_counts, q, s);
  LO_LAUNCH_OK("silu_mul_token_quant_kernel");
  return LO_OK;
}

}  // namespace lo

extern "C" int lo_per_token_quant_int8(const void *x, int x_dtype, int64_t M, int64_t K, int8_t *q, float *s,
                                       void *stream) {
  using namespace lo;
  LO_REQUIRE(M >= 0, "per-token quant: negative row count");
  if (M == 0) return LO_OK;
  LO_REQUIRE(x && q && s, "per-token quant: null pointer");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
             "per-token quant: x must be 16-byte and q 8-byte aligned");
  return launch_token_quant(x, x_dtype, M, K, 0, nullptr, q, s, static_cast<cudaStream_t>(stream));
}

extern "C" int lo_silu_mul_quant_int8(const void *input, int64_t rows, int64_t d, int8_t *q, float *s, void *stream) {
  using namespace lo;
  LO_REQUIRE(rows >= 0, "silu-mul quant: negative row count");
  if (rows == 0) return LO_OK;
  LO_REQUIRE(input && q && s, "silu-mul quant: null pointer");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(input) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
             "silu-mul quant: input must be 16-byte and q 8-byte aligned");
  return launch_silu_mul_token_quant(input, rows, d, nullptr, 0, nullptr, q, s, static_cast<cudaStream_t>(stream));
}

extern "C" int lo_silu_mul_quant_int8_masked(const void *input, int64_t groups, int64_t group_rows, int64_t d,
                                             const int32_t *tokens_per_group, int8_t *q, float *s, void *stream) {
  using namespace lo;
  LO_REQUIRE(groups >= 0 && group_rows >= 0, "silu-mul quant: negative shape");
  if (groups * group_rows == 0) return LO_OK;
  LO_REQUIRE(input && q && s, "silu-mul quant: null pointer");
  LO_REQUIRE((reinterpret_cast<uintptr_t>(input) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
             "silu-mul quant: input must be 16-byte and q 8-byte aligned");
  return launch_silu_mul_token_quant(input, groups * group_rows, d, nullptr, 0, nullptr, q, s,
                                     static_cast<cudaStream_t>(stream), group_rows, tokens_per_group);
}

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
