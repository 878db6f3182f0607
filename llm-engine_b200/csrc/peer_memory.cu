// Set-up helpers for the head-sharded exchange (include/pkv.h, "head-sharded decode"): device buffers that
// the other GPUs of the box can store into.  One process per GPU: a rank allocates its buffer,
// hands the 64-byte handle to the other ranks by whatever channel the caller has (the bench and
// the tests use torch.distributed), and every rank opens every other rank's handle.  These four
// functions are the only ones of the library that allocate or map device memory; they run once,
// before the serving loop.
#include <cuda_runtime.h>

#include <cstring>

#include "status.hpp"

extern "C" {

int pkv_peer_alloc(size_t bytes, void** ptr, void* handle64) {
  using namespace pkv;
  if (!ptr || !handle64 || bytes == 0) return fail(PKV_E_ARG, "pkv_peer_alloc: null output or zero size");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return fail(PKV_E_CUDA, "pkv_peer_alloc: cudaMalloc of %zu bytes: %s", bytes, cudaGetErrorString(e));
  e = cudaMemset(p, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(PKV_E_CUDA, "pkv_peer_alloc: %s", cudaGetErrorString(e));
  }
  std::memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return PKV_OK;
}

int pkv_peer_open(const void* handle64, void** ptr) {
  using namespace pkv;
  if (!handle64 || !ptr) return fail(PKV_E_ARG, "pkv_peer_open: null pointer");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(PKV_E_CUDA, "pkv_peer_open: %s", cudaGetErrorString(e));
  *ptr = p;
  return PKV_OK;
}

int pkv_peer_close(void* ptr) {
  using namespace pkv;
  if (!ptr) return PKV_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return fail(PKV_E_CUDA, "pkv_peer_close: %s", cudaGetErrorString(e));
  return PKV_OK;
}

int pkv_peer_free(void* ptr) {
  using namespace pkv;
  if (!ptr) return PKV_OK;
  const cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return fail(PKV_E_CUDA, "pkv_peer_free: %s", cudaGetErrorString(e));
  return PKV_OK;
}

}  // extern "C"
