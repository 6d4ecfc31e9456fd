// Set-up calls for memory that other processes on the node map (CUDA IPC): the receive buffers and flag words of the
// GEMM + all-reduce exchange.  Host code only; these are the only entry points of the library that allocate.
#include <string.h>

#include "common.cuh"

using namespace sglb;

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI passes IPC handles as 64 bytes");

extern "C" int sglb200_peer_alloc(int64_t bytes, void** dev_ptr, unsigned char* handle64) {
  SGLB_REQUIRE(bytes > 0 && dev_ptr && handle64, SGLB200_ERR_NULL, "bytes=%lld, dev_ptr and handle64 must be given",
               (long long)bytes);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaMalloc(%lld): %s", (long long)bytes, cudaGetErrorString(e));
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(SGLB200_ERR_LAUNCH, "peer_alloc: %s", cudaGetErrorString(e));
  }
  memcpy(handle64, &h, 64);
  *dev_ptr = p;
  return SGLB200_OK;
}

extern "C" int sglb200_peer_open(const unsigned char* handle64, void** dev_ptr) {
  SGLB_REQUIRE(handle64 && dev_ptr, SGLB200_ERR_NULL, "handle64 and dev_ptr must be given");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  *dev_ptr = p;
  return SGLB200_OK;
}

extern "C" int sglb200_peer_close(void* dev_ptr) {
  if (!dev_ptr) return SGLB200_OK;
  cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
  if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
  return SGLB200_OK;
}

extern "C" int sglb200_peer_free(void* dev_ptr) {
  if (!dev_ptr) return SGLB200_OK;
  cudaError_t e = cudaFree(dev_ptr);
  if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaFree: %s", cudaGetErrorString(e));
  return SGLB200_OK;
}
