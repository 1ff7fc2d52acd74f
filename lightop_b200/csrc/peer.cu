// Device buffers that the other ranks of a node can write: allocation, export as an inter-process handle and
// mapping of a peer's handle.  Expert parallelism uses them as landing zones: the dispatch kernel stores its
// records straight into the destination rank's receive buffer and the down GEMM stores its output rows straight
// into the source rank's return buffer, both with plain stores over NVLink.  Nothing here loads from a peer.
#include "common.h"
#include <cstring>

namespace lo {
namespace {
__global__ void words_to_host_kernel(const int32_t *__restrict__ src, volatile int32_t *__restrict__ dst, int64_t n) {
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
  __threadfence_system();
}
}  // namespace
}  // namespace lo

// A few words from device memory into page-locked host memory, written by a kernel instead of a copy engine: a copy
// engine takes its transfers in order, so a small read queued behind a large device-to-host transfer of another
// stream waits for all of it.  `dst_host` is page-locked memory that the device can address (cudaHostAlloc or
// cudaHostRegister under unified addressing); the words are there once the stream has reached the kernel's end.
extern "C" int lo_words_to_host(const int32_t *src, int32_t *dst_host, int64_t n, void *stream) {
  using namespace lo;
  LO_REQUIRE(n >= 0 && n <= (1 << 20), "words_to_host: bad count");
  if (n == 0) return LO_OK;
  LO_REQUIRE(src && dst_host, "words_to_host: null pointer");
  words_to_host_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(src, dst_host, n);
  LO_LAUNCH_OK("words_to_host_kernel");
  return LO_OK;
}

extern "C" int lo_peer_alloc(size_t bytes, void **ptr) {
  using namespace lo;
  LO_REQUIRE(ptr != nullptr && bytes > 0, "peer_alloc: bad argument");
  *ptr = nullptr;
  // a plain device allocation of its own: the handle then names exactly this buffer, at offset 0
  LO_CUDA_OK(cudaMalloc(ptr, bytes));
  return LO_OK;
}

extern "C" int lo_peer_free(void *ptr) {
  using namespace lo;
  if (ptr == nullptr) return LO_OK;
  LO_CUDA_OK(cudaFree(ptr));
  return LO_OK;
}

extern "C" int lo_peer_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

extern "C" int lo_peer_export(const void *ptr, uint8_t *handle) {
  using namespace lo;
  LO_REQUIRE(ptr != nullptr && handle != nullptr, "peer_export: null pointer");
  cudaIpcMemHandle_t h;
  LO_CUDA_OK(cudaIpcGetMemHandle(&h, const_cast<void *>(ptr)));
  memcpy(handle, &h, sizeof(h));
  return LO_OK;
}

extern "C" int lo_peer_open(const uint8_t *handle, void **ptr) {
  using namespace lo;
  LO_REQUIRE(ptr != nullptr && handle != nullptr, "peer_open: null pointer");
  *ptr = nullptr;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  LO_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return LO_OK;
}

extern "C" int lo_peer_close(void *ptr) {
  using namespace lo;
  if (ptr == nullptr) return LO_OK;
  LO_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return LO_OK;
}
