// Host-side construction of TMA tensor maps, and the device-side mbarrier / bulk
// tensor copy primitives the kernels share.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <cstdint>

#include "status.hpp"

namespace pkv {

// cuTensorMapEncodeTiled is a driver entry point; it is looked up through the
// runtime so the library needs no link-time dependency on libcuda.
inline PFN_cuTensorMapEncodeTiled tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
  }();
  return fn;
}

// A K or V pool viewed as a 2-D tensor [rows = slots][cols = kv_dim] of 16-bit
// elements, fetched in boxes of box_rows x 64 columns (128 bytes) with the
// 128-byte swizzle, so that consecutive rows of a box land in different
// shared-memory banks for ldmatrix.  The pool's slot count is not part of the
// launcher signature; rows is therefore an upper bound used only for the
// hardware's out-of-bounds check and block tables must name real blocks.
inline int make_pool_tensor_map(CUtensorMap* map, const void* pool, bool is_bf16, int kv_dim, uint32_t box_rows,
                                uint64_t rows_bound) {
  PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
  if (!enc) return fail(PKV_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(kv_dim), rows_bound};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(kv_dim) * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                         const_cast<void*>(pool), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PKV_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return PKV_OK;
}

#if defined(__CUDACC__)
// ---- mbarrier ---------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// One lane arrives for its whole warp (count 32): call after __syncwarp().  Thirty-two lanes arriving
// on one barrier word one by one serialise in the shared-memory pipe and delay the warp's next
// shared-memory operation by a couple of hundred cycles.
__device__ __forceinline__ void mbar_arrive_warp(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], 32;\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking look at a phase: a few tens of cycles, where try_wait costs a few hundred even
// when the phase has long completed.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: a quick look first, then up to `limit` blocking polls (each blocks for a
// hardware-defined time slice); reports failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 17)) {
  if (mbar_test(bar, parity)) return true;
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// Bounded busy wait for a single latency-critical thread: it never sleeps, so it sees the phase
// flip within one poll.
__device__ __forceinline__ bool mbar_spin(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 22)) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_test(bar, parity)) return true;
  return false;
}
// ---- TMA: one box of a 2-D tensor map into this block's shared memory ---------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(dst),
      "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void movmatrix_trans(uint32_t& dst, uint32_t src) {
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(dst) : "r"(src));
}
#endif

}  // namespace pkv
