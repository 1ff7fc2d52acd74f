// A host with no Python and no torch drives the fused block-INT8 MoE layer through the C ABI:
// it reads the operands from a binary file, allocates device memory with the CUDA runtime, calls
// lo_topk_softmax and lo_fused_moe_block_int8 from the shared library (loaded with dlopen, bound by
// name as a foreign-function interface would), and writes the output rows to a second file.
//
//   host_moe <liblightop_b200.so> <input.bin> <output.bin>
//
// input.bin (little endian): int64 M, E, k, H, I; then logits f32 [M,E], x bf16 [M,H],
// w1 int8 [E,2I,H], w2 int8 [E,H,I], w1_scale f32 [E,2I/128,H/128], w2_scale f32 [E,H/128,I/128].
// output.bin: topk_ids i32 [M,k], topk_weights f32 [M,k], y bf16 [M,H].
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../include/lightop_b200.h"

#define CHECK_CUDA(x)                                                                   \
  do {                                                                                  \
    cudaError_t e_ = (x);                                                               \
    if (e_ != cudaSuccess) {                                                            \
      std::fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_));              \
      return 2;                                                                         \
    }                                                                                   \
  } while (0)

template <typename F> static F sym(void *lib, const char *name) {
  void *p = dlsym(lib, name);
  if (!p) {
    std::fprintf(stderr, "missing symbol %s\n", name);
    std::exit(3);
  }
  return reinterpret_cast<F>(p);
}

template <typename T> static bool read_vec(FILE *f, std::vector<T> &v, size_t n) {
  v.resize(n);
  return std::fread(v.data(), sizeof(T), n, f) == n;
}

template <typename T> static T *to_device(const std::vector<T> &v) {
  T *d = nullptr;
  if (cudaMalloc(&d, v.size() * sizeof(T)) != cudaSuccess) return nullptr;
  if (cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
  return d;
}

int main(int argc, char **argv) {
  if (argc != 4) {
    std::fprintf(stderr, "usage: %s <library> <input.bin> <output.bin>\n", argv[0]);
    return 1;
  }
  void *lib = dlopen(argv[1], RTLD_NOW);
  if (!lib) {
    std::fprintf(stderr, "dlopen: %s\n", dlerror());
    return 3;
  }
  auto topk = sym<decltype(&lo_topk_softmax)>(lib, "lo_topk_softmax");
  auto ws_bytes = sym<decltype(&lo_fused_moe_workspace_bytes)>(lib, "lo_fused_moe_workspace_bytes");
  auto fused = sym<decltype(&lo_fused_moe_block_int8)>(lib, "lo_fused_moe_block_int8");
  auto last_error = sym<decltype(&lo_last_error)>(lib, "lo_last_error");

  FILE *f = std::fopen(argv[2], "rb");
  if (!f) return 1;
  int64_t dims[5];
  if (std::fread(dims, sizeof(int64_t), 5, f) != 5) return 1;
  const int64_t M = dims[0], E = dims[1], k = dims[2], H = dims[3], I = dims[4];
  std::vector<float> logits, w1s, w2s;
  std::vector<uint16_t> x;
  std::vector<int8_t> w1, w2;
  if (!read_vec(f, logits, M * E) || !read_vec(f, x, M * H) || !read_vec(f, w1, E * 2 * I * H) || !read_vec(f, w2, E * H * I) ||
      !read_vec(f, w1s, E * (2 * I / 128) * (H / 128)) || !read_vec(f, w2s, E * (H / 128) * (I / 128)))
    return 1;
  std::fclose(f);

  float *d_logits = to_device(logits), *d_w1s = to_device(w1s), *d_w2s = to_device(w2s);
  uint16_t *d_x = to_device(x);
  int8_t *d_w1 = to_device(w1), *d_w2 = to_device(w2);
  if (!d_logits || !d_w1s || !d_w2s || !d_x || !d_w1 || !d_w2) return 2;
  float *d_tw = nullptr;
  int32_t *d_ti = nullptr, *d_status = nullptr;
  uint16_t *d_cache3 = nullptr, *d_y = nullptr;
  void *d_ws = nullptr;
  const size_t nws = ws_bytes(M, (int)E, (int)E, (int)k, H, I);
  CHECK_CUDA(cudaMalloc(&d_tw, M * k * sizeof(float)));
  CHECK_CUDA(cudaMalloc(&d_ti, M * k * sizeof(int32_t)));
  CHECK_CUDA(cudaMalloc(&d_status, sizeof(int32_t)));
  CHECK_CUDA(cudaMemset(d_status, 0, sizeof(int32_t)));
  CHECK_CUDA(cudaMalloc(&d_cache3, M * k * H * sizeof(uint16_t)));
  CHECK_CUDA(cudaMalloc(&d_y, M * H * sizeof(uint16_t)));
  CHECK_CUDA(cudaMalloc(&d_ws, nws));
  cudaStream_t stream;
  CHECK_CUDA(cudaStreamCreate(&stream));

  int rc = topk(d_logits, LO_F32, M, (int)E, (int)k, 1, d_tw, d_ti, LO_I32, nullptr, stream);
  if (rc == 0)
    rc = fused(d_x, d_w1, d_w2, d_w1s, d_w2s, d_tw, d_ti, LO_I32, nullptr, (int)E, M, (int)E, (int)k, H, I, d_cache3, nullptr,
               d_y, 0, 1.0f, d_ws, nws, d_status, stream);
  if (rc != 0) {
    std::fprintf(stderr, "library call failed (%d): %s\n", rc, last_error());
    return 4;
  }
  CHECK_CUDA(cudaStreamSynchronize(stream));
  int32_t status = -1;
  CHECK_CUDA(cudaMemcpy(&status, d_status, sizeof(status), cudaMemcpyDeviceToHost));
  if (status != 0) {
    std::fprintf(stderr, "a bounded wait ran out on the device (waiter %d)\n", status);
    return 5;
  }
  std::vector<int32_t> ti(M * k);
  std::vector<float> tw(M * k);
  std::vector<uint16_t> y(M * H);
  CHECK_CUDA(cudaMemcpy(ti.data(), d_ti, ti.size() * sizeof(int32_t), cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(tw.data(), d_tw, tw.size() * sizeof(float), cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(y.data(), d_y, y.size() * sizeof(uint16_t), cudaMemcpyDeviceToHost));
  FILE *o = std::fopen(argv[3], "wb");
  if (!o) return 1;
  std::fwrite(ti.data(), sizeof(int32_t), ti.size(), o);
  std::fwrite(tw.data(), sizeof(float), tw.size(), o);
  std::fwrite(y.data(), sizeof(uint16_t), y.size(), o);
  std::fclose(o);
  std::printf("ok M=%lld E=%lld k=%lld H=%lld I=%lld workspace=%zu\n", (long long)M, (long long)E, (long long)k, (long long)H,
              (long long)I, nws);
  return 0;
}
