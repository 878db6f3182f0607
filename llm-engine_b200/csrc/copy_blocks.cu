// Prefix-cache copy-on-write block copy (include/pkv.h, "block copy").
//
// A block of one pool is block_size * kv_dim elements of contiguous memory, so the
// copy of pair (src, dst) in pool p is a straight 16-byte-vector memcpy of
// block_bytes.  grid = (pieces of a block, pairs, pools): every (pair, pool) gets
// its own thread blocks and every thread keeps four independent 16-byte loads in
// flight.  Bit-exact by construction.
#include "common.cuh"
#include "launch_util.hpp"
#include "status.hpp"

namespace pkv {
namespace {

constexpr int kCopyThreads = 128;
constexpr int kCopyUnroll = 4;

struct TwoPools { void* p[2]; };

template <bool FROM_ARRAY>
__global__ void __launch_bounds__(kCopyThreads) copy_blocks_kernel(TwoPools two, void* const* __restrict__ pools,
                                                                    const int* __restrict__ pairs, int block_vecs) {
  char* pool = static_cast<char*>(FROM_ARRAY ? pools[blockIdx.z] : two.p[blockIdx.z]);
  const int src = __ldg(pairs + 2 * blockIdx.y), dst = __ldg(pairs + 2 * blockIdx.y + 1);
  if (src == dst) return;
  const uint4* s = reinterpret_cast<const uint4*>(pool) + static_cast<size_t>(src) * block_vecs;
  uint4* d = reinterpret_cast<uint4*>(pool) + static_cast<size_t>(dst) * block_vecs;
  const int base = blockIdx.x * kCopyThreads * kCopyUnroll + threadIdx.x;
  uint4 r[kCopyUnroll];
#pragma unroll
  for (int u = 0; u < kCopyUnroll; ++u) {
    const int i = base + u * kCopyThreads;
    if (i < block_vecs) r[u] = ld_nc_u4(s + i);
  }
#pragma unroll
  for (int u = 0; u < kCopyUnroll; ++u) {
    const int i = base + u * kCopyThreads;
    if (i < block_vecs) d[i] = r[u];
  }
}

// Blocks whose byte size or pool address is not 16-byte granular.
template <bool FROM_ARRAY>
__global__ void __launch_bounds__(kCopyThreads) copy_blocks_bytes_kernel(TwoPools two, void* const* __restrict__ pools,
                                                                          const int* __restrict__ pairs, size_t block_bytes) {
  char* pool = static_cast<char*>(FROM_ARRAY ? pools[blockIdx.z] : two.p[blockIdx.z]);
  const int src = pairs[2 * blockIdx.y], dst = pairs[2 * blockIdx.y + 1];
  if (src == dst) return;
  const char* s = pool + static_cast<size_t>(src) * block_bytes;
  char* d = pool + static_cast<size_t>(dst) * block_bytes;
  for (size_t i = blockIdx.x * static_cast<size_t>(kCopyThreads) + threadIdx.x; i < block_bytes;
       i += static_cast<size_t>(gridDim.x) * kCopyThreads)
    d[i] = s[i];
}

int copy_impl(TwoPools two, void* const* pools, int n_pools, bool pools_aligned, const int* pairs, int n_pairs,
              size_t block_bytes, pkv_stream stream) {
  if (n_pairs <= 0 || n_pools <= 0 || block_bytes == 0) return PKV_OK;
  if (!pairs) return fail(PKV_E_ARG, "pkv_copy_blocks: null pair list");
  if (n_pairs > 65535 || n_pools > 65535)
    return fail(PKV_E_UNSUPPORTED, "pkv_copy_blocks: at most 65535 pairs and 65535 pools per call (got %d, %d)", n_pairs, n_pools);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (block_bytes % 16 == 0 && pools_aligned) {
    const int block_vecs = static_cast<int>(block_bytes / 16);
    const int per_cta = kCopyThreads * kCopyUnroll;
    dim3 grid((block_vecs + per_cta - 1) / per_cta, n_pairs, n_pools);
    if (pools) copy_blocks_kernel<true><<<grid, kCopyThreads, 0, s>>>(two, pools, pairs, block_vecs);
    else copy_blocks_kernel<false><<<grid, kCopyThreads, 0, s>>>(two, pools, pairs, block_vecs);
    return check_launch("copy_blocks_kernel");
  }
  dim3 grid(static_cast<unsigned>((block_bytes + kCopyThreads * 8 - 1) / (kCopyThreads * 8)), n_pairs, n_pools);
  if (pools) copy_blocks_bytes_kernel<true><<<grid, kCopyThreads, 0, s>>>(two, pools, pairs, block_bytes);
  else copy_blocks_bytes_kernel<false><<<grid, kCopyThreads, 0, s>>>(two, pools, pairs, block_bytes);
  return check_launch("copy_blocks_bytes_kernel");
}

int copy_two(void* k_cache, void* v_cache, const int* pairs, int n_pairs, int block_size, int kv_dim, size_t elem,
             pkv_stream stream) {
  if (n_pairs <= 0) return PKV_OK;
  if (!k_cache || !v_cache) return fail(PKV_E_ARG, "pkv_copy_blocks: null pool pointer");
  if (block_size <= 0 || kv_dim <= 0) return fail(PKV_E_ARG, "pkv_copy_blocks: block_size %d, kv_dim %d must be > 0", block_size, kv_dim);
  TwoPools two{{k_cache, v_cache}};
  return copy_impl(two, nullptr, 2, aligned16(k_cache) && aligned16(v_cache), pairs, n_pairs,
                   elem * static_cast<size_t>(block_size) * kv_dim, stream);
}

}  // namespace
}  // namespace pkv

extern "C" {
int pkv_copy_blocks_f16(void* k_cache, void* v_cache, const int* src_dst_pairs, int n_pairs, int block_size,
                        int kv_dim, pkv_stream stream) {
  return pkv::copy_two(k_cache, v_cache, src_dst_pairs, n_pairs, block_size, kv_dim, 2, stream);
}
int pkv_copy_blocks_bf16(void* k_cache, void* v_cache, const int* src_dst_pairs, int n_pairs, int block_size,
                         int kv_dim, pkv_stream stream) {
  return pkv::copy_two(k_cache, v_cache, src_dst_pairs, n_pairs, block_size, kv_dim, 2, stream);
}
int pkv_copy_blocks_f32(void* k_cache, void* v_cache, const int* src_dst_pairs, int n_pairs, int block_size,
                        int kv_dim, pkv_stream stream) {
  return pkv::copy_two(k_cache, v_cache, src_dst_pairs, n_pairs, block_size, kv_dim, 4, stream);
}
// The pool base pointers live in device memory, so their alignment cannot be
// inspected here: every pool must be 16-byte aligned when block_bytes is a
// multiple of 16 (cudaMalloc'd pools always are).
int pkv_copy_blocks_layers(void* const* d_cache_ptrs, int n_caches, const int* src_dst_pairs, int n_pairs,
                           size_t block_bytes, pkv_stream stream) {
  if (n_pairs <= 0 || n_caches <= 0) return PKV_OK;
  if (!d_cache_ptrs) return pkv::fail(PKV_E_ARG, "pkv_copy_blocks_layers: null pool pointer array");
  pkv::TwoPools two{{nullptr, nullptr}};
  return pkv::copy_impl(two, d_cache_ptrs, n_caches, true, src_dst_pairs, n_pairs, block_bytes, stream);
}
}
