// Launch-time error capture shared by the CUDA entry points.
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>

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

// Programmatic dependent launch: the kernel may be scheduled while its predecessor
// on the stream is still running; it must call pdl_wait() before it reads anything
// the predecessor (or anything before that) wrote, which blocks until the
// predecessor has completed and flushed.  What is gained is the launch latency and
// the on-chip prologue of every kernel in a chain of short launches (append ->
// attention -> merge, once per layer).  PKV_PDL=0 turns it off.
inline bool pdl_enabled() {
  static const bool on = [] { const char* e = std::getenv("PKV_PDL"); return !(e && *e == '0'); }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#if defined(__CUDACC__)
// Device side of the above.  Both are no-ops when the kernel was launched without
// the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
#endif

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace pkv
