// K/V append (include/pkv.h, "K/V append"): scatter each new token's K and V row to
// row slots[t] of the block pool.  A pure byte copy, so one kernel serves every
// element type; the dtype-suffixed entry points only fix the row size.
//
// Work is laid out as a flat list of 16-byte pieces over (token, K|V, piece), so a
// warp moves 512 contiguous bytes of one row per instruction and the grid scales
// with the step size (8 tokens for a small decode batch, 16 Ki for a prefill chunk)
// instead of one thread block per token with scalar 2-byte stores
// (src/kernels/store_kv.cu:20-29).
#include "common.cuh"
#include "launch_util.hpp"
#include "status.hpp"

namespace pkv {
namespace {

constexpr int kAppendThreads = 256;

__global__ void __launch_bounds__(kAppendThreads) append_vec16_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v,
                                                                       const int* __restrict__ slots, uint4* __restrict__ k_cache,
                                                                       uint4* __restrict__ v_cache, long long total, int row_vecs) {
  pdl_launch_dependents();
  pdl_wait();
  // piece index -> (token, which pool, 16-byte piece of the row)
  for (long long i = blockIdx.x * static_cast<long long>(kAppendThreads) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kAppendThreads) {
    const long long row = i / row_vecs;
    const int piece = static_cast<int>(i - row * row_vecs);
    const int token = static_cast<int>(row >> 1);
    const bool is_v = row & 1;
    const long long dst = static_cast<long long>(__ldg(slots + token)) * row_vecs + piece;
    const long long src = static_cast<long long>(token) * row_vecs + piece;
    if (is_v) v_cache[dst] = ld_nc_u4(v + src);
    else k_cache[dst] = ld_nc_u4(k + src);
  }
}

// Rows whose size or base address is not a multiple of 16 bytes: element-wise.
template <typename W>
__global__ void __launch_bounds__(kAppendThreads) append_scalar_kernel(const W* __restrict__ k, const W* __restrict__ v,
                                                                        const int* __restrict__ slots, W* __restrict__ k_cache,
                                                                        W* __restrict__ v_cache, int kv_dim) {
  pdl_launch_dependents();
  pdl_wait();
  const int token = blockIdx.x;
  const size_t src = static_cast<size_t>(token) * kv_dim, dst = static_cast<size_t>(slots[token]) * kv_dim;
  for (int d = threadIdx.x; d < kv_dim; d += kAppendThreads) {
    k_cache[dst + d] = k[src + d];
    v_cache[dst + d] = v[src + d];
  }
}

template <typename W>
int append_impl(const void* k, const void* v, const int* slots, void* k_cache, void* v_cache, int n_tokens,
                int kv_dim, pkv_stream stream) {
  if (n_tokens <= 0 || kv_dim <= 0) return PKV_OK;  // as src/kernels/store_kv.cu:34
  if (!k || !v || !slots || !k_cache || !v_cache) return fail(PKV_E_ARG, "pkv_append: null device pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t row_bytes = sizeof(W) * static_cast<size_t>(kv_dim);
  if (row_bytes % 16 == 0 && aligned16(k) && aligned16(v) && aligned16(k_cache) && aligned16(v_cache)) {
    const int row_vecs = static_cast<int>(row_bytes / 16);
    const long long total = 2ll * n_tokens * row_vecs;
    long long blocks = (total + kAppendThreads - 1) / kAppendThreads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    launch_pdl(append_vec16_kernel, dim3(static_cast<unsigned>(blocks)), dim3(kAppendThreads), 0, s,
               static_cast<const uint4*>(k), static_cast<const uint4*>(v), slots, static_cast<uint4*>(k_cache),
               static_cast<uint4*>(v_cache), total, row_vecs);
    return check_launch("append_vec16_kernel");
  }
  launch_pdl(append_scalar_kernel<W>, dim3(n_tokens), dim3(kAppendThreads), 0, s, static_cast<const W*>(k),
             static_cast<const W*>(v), slots, static_cast<W*>(k_cache), static_cast<W*>(v_cache), kv_dim);
  return check_launch("append_scalar_kernel");
}

}  // namespace
}  // namespace pkv

extern "C" {
int pkv_append_f16(const void* k, const void* v, const int* slots, void* k_cache, void* v_cache, int n_tokens,
                   int kv_dim, pkv_stream stream) {
  return pkv::append_impl<uint16_t>(k, v, slots, k_cache, v_cache, n_tokens, kv_dim, stream);
}
int pkv_append_bf16(const void* k, const void* v, const int* slots, void* k_cache, void* v_cache, int n_tokens,
                    int kv_dim, pkv_stream stream) {
  return pkv::append_impl<uint16_t>(k, v, slots, k_cache, v_cache, n_tokens, kv_dim, stream);
}
int pkv_append_f32(const void* k, const void* v, const int* slots, void* k_cache, void* v_cache, int n_tokens,
                   int kv_dim, pkv_stream stream) {
  return pkv::append_impl<uint32_t>(k, v, slots, k_cache, v_cache, n_tokens, kv_dim, stream);
}
}
