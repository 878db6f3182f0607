// Launch-time error capture shared by the CUDA entry points.
#pragma once
#include <cuda_runtime.h>

#include "status.hpp"

namespace pkv {

// Reports a launch that the runtime rejected (bad configuration, no device, ...).
// Faults inside a running kernel surface later, at the caller's own
// synchronisation point, exactly as with the reference launchers.
inline int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(PKV_E_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return PKV_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace pkv
