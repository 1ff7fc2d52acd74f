// Stand-alone micro-benchmark (not part of the library): the tensor-core ceiling of the grouped GEMM.
// One thread per CTA issues tcgen05.mma M=128, K=32 kind::i8 (and kind::f8f6f4 for comparison) back to
// back on fixed shared-memory tiles, 148 CTAs, for N = 16..256; prints cycles per MMA and the implied
// all-SM rate.  This is the INT8 tensor peak the roofline discussion needs and the per-instruction
// floor (about 96 cycles for N <= 128) that bounds the kernel's MMA warp.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o bench_mma_peak lightop_b200/csrc/bench_mma_peak.cu && ./bench_mma_peak
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0; d |= (uint64_t)((saddr & 0x3ffffu) >> 4); d |= (uint64_t)1 << 16; d |= (uint64_t)(1024 >> 4) << 32; d |= (uint64_t)1 << 46; d |= (uint64_t)2 << 61; return d; }
__device__ __forceinline__ uint32_t make_idesc_i8(uint32_t n) { return (2u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24); }
__device__ __forceinline__ uint32_t make_idesc_f8(uint32_t n) { return (1u << 4) | (0u << 7) | (0u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24); }
template <int KIND>
__global__ void __launch_bounds__(128, 1) k(int iters, int n, int chains, long long *out) {
  extern __shared__ uint8_t raw[];
  uint8_t *sm = (uint8_t *)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar; __shared__ uint32_t tbase;
  for (int i = threadIdx.x; i < 64 * 1024; i += blockDim.x) sm[i] = (uint8_t)(i * 7 + 1);
  if (threadIdx.x == 0) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar))); asm volatile("fence.mbarrier_init.release.cluster;"); }
  if (threadIdx.x < 32) { asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&tbase))); asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;"); }
  asm volatile("fence.proxy.async.shared::cta;");
  asm volatile("tcgen05.fence::before_thread_sync;"); __syncthreads(); asm volatile("tcgen05.fence::after_thread_sync;");
  const uint32_t tb = tbase;
  long long t0 = 0, t1 = 0;
  if (threadIdx.x == 0) {
    const uint64_t ad = make_smem_desc(smem_u32(sm)), bd = make_smem_desc(smem_u32(sm + 16384));
    const uint32_t id = KIND == 0 ? make_idesc_i8(n) : make_idesc_f8(n);
    t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      for (int c = 0; c < chains; ++c) {
        const uint32_t d = tb + c * (512 / chains);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          if (KIND == 0) asm volatile("{.reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;}" ::"r"(d), "l"(ad + k4 * 2), "l"(bd + k4 * 2), "r"(id), "r"(k4 > 0 ? 1 : 0) : "memory");
          else asm volatile("{.reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;}" ::"r"(d), "l"(ad + k4 * 2), "l"(bd + k4 * 2), "r"(id), "r"(k4 > 0 ? 1 : 0) : "memory");
        }
      }
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
    uint32_t ok = 0; long long guard = clock64();
    while (!ok && clock64() - guard < 4000000000ll) asm volatile("{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0; selp.u32 %0,1,0,p;}" : "=r"(ok) : "r"(smem_u32(&bar)) : "memory");
    t1 = clock64();
    out[blockIdx.x] = t1 - t0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;"); __syncthreads();
  if (threadIdx.x < 32) { asm volatile("tcgen05.fence::after_thread_sync;"); asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tb)); }
}
int main() {
  // MMA-only loop on every SM: the ceiling of the tensor pipe for kind::i8 (and kind::f8f6f4) at M=128, K=32 and
  // N = 16..256, with one or two independent accumulator chains.  Prints one line per case and, last, one JSON
  // line with the all-SM rates timed with CUDA events (bench.py reads it).
  long long *d; cudaMalloc(&d, 148 * 8); long long h[148];
  cudaFuncSetAttribute(k<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 70 * 1024);
  cudaFuncSetAttribute(k<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 70 * 1024);
  int sms = 0; cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  if (sms <= 0 || sms > 148) sms = 148;
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  int ns[] = {16, 32, 64, 128, 256};
  double pops_i8_128 = 0, pops_i8_256 = 0;
  for (int kind = 0; kind < 2; ++kind) for (int ch = 1; ch <= 2; ++ch) for (int ni = 0; ni < 5; ++ni) {
    int n = ns[ni]; if (n * ch > 512) continue; int iters = 2000;
    if (kind == 0) k<0><<<sms, 128, 70 * 1024>>>(200, n, ch, d); else k<1><<<sms, 128, 70 * 1024>>>(200, n, ch, d);   // warm-up
    cudaEventRecord(e0);
    if (kind == 0) k<0><<<sms, 128, 70 * 1024>>>(iters, n, ch, d); else k<1><<<sms, 128, 70 * 1024>>>(iters, n, ch, d);
    cudaEventRecord(e1);
    cudaError_t e = cudaDeviceSynchronize(); cudaMemcpy(h, d, 148 * 8, cudaMemcpyDeviceToHost);
    float ms = 0; cudaEventElapsedTime(&ms, e0, e1);
    double cyc = (double)h[0] / (iters * ch * 4);
    double pops = 2.0 * 128 * n * 32 * (double)iters * ch * 4 * sms / (ms * 1e-3) / 1e15;
    if (kind == 0 && n == 128 && pops > pops_i8_128) pops_i8_128 = pops;
    if (kind == 0 && n == 256 && pops > pops_i8_256) pops_i8_256 = pops;
    printf("%s chains=%d N=%3d: %.1f cycles per M128xN%dxK32 MMA -> %.0f MAC/clk/SM, all-SM %.2f POPS by CUDA events  (%s)\n", kind ? "f8f6f4" : "i8    ", ch, n, cyc, n, 128.0 * n * 32 / cyc, pops, cudaGetErrorString(e));
  }
  printf("{\"int8_pops_n128\": %.4f, \"int8_pops_n256\": %.4f, \"sms\": %d}\n", pops_i8_128, pops_i8_256, sms);
  return 0;
}
