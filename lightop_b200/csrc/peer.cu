// Device buffers that the other ranks of a node can write: allocation, export as an inter-process handle and
// mapping of a peer's handle.  Expert parallelism uses them as landing zones: the dispatch kernel stores its
// records straight into the destination rank's receive buffer and the down GEMM stores its output rows straight
// into the source rank's return buffer, both with plain stores over NVLink.  Nothing here loads from a peer.
#include "common.h"
#include <cstring>

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
