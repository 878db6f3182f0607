// RoPE fused into the K/V append (include/pkv.h, "RoPE + append").
//
// llm-engine runs three launches per layer here: rope(q), rope(k), store_kv
// (src/model/cuda/cuda_model.cu:366-368; the fusion is the first item of its own
// kernel plan, src/kernels/store_kv.cu:9-12).  This kernel does all three in one pass:
// q is rotated in place, k is rotated on its way into the pool (read once, written
// once, straight to its slot), v is copied to its slot.
//
// Arithmetic is the reference's (include/engine/ops.h:56-68, src/kernels/rope.cu:32-51):
// rotate_half pairing (element i with i + head_dim/2), fp32 cos/sin tables indexed by the
// token's absolute position, x' = a*c - b*s and b*c + a*s evaluated in fp32 with separately
// rounded products (no fused multiply-add, so the result is bit-identical to the CPU code),
// then rounded to the element type.
#include "common.cuh"
#include "launch_util.hpp"
#include "status.hpp"

namespace pkv {
namespace {

constexpr int kRopeThreads = 256;

template <typename T> struct Vec16 { static constexpr int kElems = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void rotate_vec(const uint4& lo, const uint4& hi, const float* c, const float* s, uint4& out_lo,
                                           uint4& out_hi) {
  constexpr int E = Vec16<T>::kElems;
  const T* a = reinterpret_cast<const T*>(&lo);
  const T* b = reinterpret_cast<const T*>(&hi);
  T* oa = reinterpret_cast<T*>(&out_lo);
  T* ob = reinterpret_cast<T*>(&out_hi);
#pragma unroll
  for (int i = 0; i < E; ++i) {
    const float x = Elem<T>::to_f32(a[i]), y = Elem<T>::to_f32(b[i]);
    oa[i] = Elem<T>::from_f32(__fsub_rn(__fmul_rn(x, c[i]), __fmul_rn(y, s[i])));
    ob[i] = Elem<T>::from_f32(__fadd_rn(__fmul_rn(y, c[i]), __fmul_rn(x, s[i])));
  }
}

// One thread per 16-byte piece: rope pieces of the q heads, rope pieces of the k heads, copy pieces of v.
template <typename T>
__global__ void __launch_bounds__(kRopeThreads) rope_append_vec_kernel(T* __restrict__ q, const T* __restrict__ k,
                                                                        const T* __restrict__ v,
                                                                        const int* __restrict__ positions,
                                                                        const float* __restrict__ cos_table,
                                                                        const float* __restrict__ sin_table,
                                                                        const int* __restrict__ slots, T* __restrict__ k_cache,
                                                                        T* __restrict__ v_cache, int n_tokens, int q_heads,
                                                                        int kv_heads, int head_dim) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int E = Vec16<T>::kElems;
  const int half = head_dim / 2;
  const int ppr = half / E;                        // rope pieces per head
  const int kv_dim = kv_heads * head_dim;
  const int v_pieces = kv_dim / E;
  const int per_token = (q_heads + kv_heads) * ppr + v_pieces;
  const long long total = static_cast<long long>(n_tokens) * per_token;
  for (long long w = blockIdx.x * static_cast<long long>(kRopeThreads) + threadIdx.x; w < total;
       w += static_cast<long long>(gridDim.x) * kRopeThreads) {
    const int token = static_cast<int>(w / per_token);
    int u = static_cast<int>(w - static_cast<long long>(token) * per_token);
    if (u >= (q_heads + kv_heads) * ppr) {           // v: plain copy to the slot
      u -= (q_heads + kv_heads) * ppr;
      const uint4* src = reinterpret_cast<const uint4*>(v + static_cast<size_t>(token) * kv_dim) + u;
      uint4* dst = reinterpret_cast<uint4*>(v_cache + static_cast<size_t>(__ldg(slots + token)) * kv_dim) + u;
      *dst = ld_nc_u4(src);
      continue;
    }
    const int head = u / ppr, piece = u - head * ppr;
    const size_t t = static_cast<size_t>(__ldg(positions + token)) * half + piece * E;
    float c[E], s[E];
#pragma unroll
    for (int i = 0; i < E; i += 4) {
      const float4 cv = __ldg(reinterpret_cast<const float4*>(cos_table + t + i));
      const float4 sv = __ldg(reinterpret_cast<const float4*>(sin_table + t + i));
      c[i] = cv.x; c[i + 1] = cv.y; c[i + 2] = cv.z; c[i + 3] = cv.w;
      s[i] = sv.x; s[i + 1] = sv.y; s[i + 2] = sv.z; s[i + 3] = sv.w;
    }
    uint4 lo, hi, olo, ohi;
    if (head < q_heads) {
      T* row = q + (static_cast<size_t>(token) * q_heads + head) * head_dim + piece * E;
      lo = *reinterpret_cast<const uint4*>(row);
      hi = *reinterpret_cast<const uint4*>(row + half);
      rotate_vec<T>(lo, hi, c, s, olo, ohi);
      *reinterpret_cast<uint4*>(row) = olo;
      *reinterpret_cast<uint4*>(row + half) = ohi;
    } else {
      const int kh = head - q_heads;
      const T* row = k + static_cast<size_t>(token) * kv_dim + kh * head_dim + piece * E;
      lo = ld_nc_u4(row);
      hi = ld_nc_u4(row + half);
      rotate_vec<T>(lo, hi, c, s, olo, ohi);
      T* dst = k_cache + static_cast<size_t>(__ldg(slots + token)) * kv_dim + kh * head_dim + piece * E;
      *reinterpret_cast<uint4*>(dst) = olo;
      *reinterpret_cast<uint4*>(dst + half) = ohi;
    }
  }
}

// Any head_dim (even), any alignment: one thread per rotation pair / per v element.
template <typename T>
__global__ void __launch_bounds__(kRopeThreads) rope_append_scalar_kernel(T* __restrict__ q, const T* __restrict__ k,
                                                                           const T* __restrict__ v,
                                                                           const int* __restrict__ positions,
                                                                           const float* __restrict__ cos_table,
                                                                           const float* __restrict__ sin_table,
                                                                           const int* __restrict__ slots, T* __restrict__ k_cache,
                                                                           T* __restrict__ v_cache, int n_tokens, int q_heads,
                                                                           int kv_heads, int head_dim) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = head_dim / 2;
  const int kv_dim = kv_heads * head_dim;
  const int per_token = (q_heads + kv_heads) * half + kv_dim;
  const long long total = static_cast<long long>(n_tokens) * per_token;
  for (long long w = blockIdx.x * static_cast<long long>(kRopeThreads) + threadIdx.x; w < total;
       w += static_cast<long long>(gridDim.x) * kRopeThreads) {
    const int token = static_cast<int>(w / per_token);
    int u = static_cast<int>(w - static_cast<long long>(token) * per_token);
    if (u >= (q_heads + kv_heads) * half) {
      u -= (q_heads + kv_heads) * half;
      v_cache[static_cast<size_t>(slots[token]) * kv_dim + u] = v[static_cast<size_t>(token) * kv_dim + u];
      continue;
    }
    const int head = u / half, i = u - head * half;
    const size_t t = static_cast<size_t>(positions[token]) * half + i;
    const float c = cos_table[t], s = sin_table[t];
    if (head < q_heads) {
      T* row = q + (static_cast<size_t>(token) * q_heads + head) * head_dim;
      const float a = Elem<T>::to_f32(row[i]), b = Elem<T>::to_f32(row[i + half]);
      row[i] = Elem<T>::from_f32(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
      row[i + half] = Elem<T>::from_f32(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s)));
    } else {
      const int kh = head - q_heads;
      const T* row = k + static_cast<size_t>(token) * kv_dim + kh * head_dim;
      const float a = Elem<T>::to_f32(row[i]), b = Elem<T>::to_f32(row[i + half]);
      T* dst = k_cache + static_cast<size_t>(slots[token]) * kv_dim + kh * head_dim;
      dst[i] = Elem<T>::from_f32(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
      dst[i + half] = Elem<T>::from_f32(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s)));
    }
  }
}

template <typename T>
int rope_append_impl(void* q, const void* k, const void* v, const int* positions, const float* cos_table,
                     const float* sin_table, const int* slots, void* k_cache, void* v_cache, int n_tokens, int q_heads,
                     int kv_heads, int head_dim, pkv_stream stream) {
  const char* fn = "pkv_rope_append";
  if (n_tokens <= 0 || head_dim <= 0 || (q_heads <= 0 && kv_heads <= 0)) return PKV_OK;  // as launch_rope / launch_store_kv
  if (q_heads < 0 || kv_heads < 0) return fail(PKV_E_ARG, "%s: negative head count", fn);
  if (head_dim % 2) return fail(PKV_E_UNSUPPORTED, "%s: head_dim %d must be even (rotation pairs)", fn, head_dim);
  if (!positions || !cos_table || !sin_table) return fail(PKV_E_ARG, "%s: null positions or tables", fn);
  if (q_heads > 0 && !q) return fail(PKV_E_ARG, "%s: null q", fn);
  if (kv_heads > 0 && (!k || !v || !slots || !k_cache || !v_cache)) return fail(PKV_E_ARG, "%s: null K/V pointer", fn);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  constexpr int E = Vec16<T>::kElems;
  const int half = head_dim / 2;
  const bool vec = half % E == 0 && half % 4 == 0 && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(k_cache) &&
                   aligned16(v_cache) && aligned16(cos_table) && aligned16(sin_table);
  const long long units = vec ? static_cast<long long>(n_tokens) * ((q_heads + kv_heads) * (half / E) + kv_heads * head_dim / E)
                              : static_cast<long long>(n_tokens) * ((q_heads + kv_heads) * half + kv_heads * head_dim);
  long long blocks = (units + kRopeThreads - 1) / kRopeThreads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (vec)
    launch_pdl(rope_append_vec_kernel<T>, dim3(static_cast<unsigned>(blocks)), dim3(kRopeThreads), 0, s, static_cast<T*>(q),
               static_cast<const T*>(k), static_cast<const T*>(v), positions, cos_table, sin_table, slots,
               static_cast<T*>(k_cache), static_cast<T*>(v_cache), n_tokens, q_heads, kv_heads, head_dim);
  else
    launch_pdl(rope_append_scalar_kernel<T>, dim3(static_cast<unsigned>(blocks)), dim3(kRopeThreads), 0, s, static_cast<T*>(q),
               static_cast<const T*>(k), static_cast<const T*>(v), positions, cos_table, sin_table, slots,
               static_cast<T*>(k_cache), static_cast<T*>(v_cache), n_tokens, q_heads, kv_heads, head_dim);
  return check_launch("rope_append_kernel");
}

}  // namespace
}  // namespace pkv

extern "C" {
int pkv_rope_append_f16(void* q, const void* k, const void* v, const int* positions, const float* cos_table,
                        const float* sin_table, const int* slots, void* k_cache, void* v_cache, int n_tokens,
                        int q_heads, int kv_heads, int head_dim, pkv_stream stream) {
  return pkv::rope_append_impl<__half>(q, k, v, positions, cos_table, sin_table, slots, k_cache, v_cache, n_tokens, q_heads,
                                       kv_heads, head_dim, stream);
}
int pkv_rope_append_bf16(void* q, const void* k, const void* v, const int* positions, const float* cos_table,
                         const float* sin_table, const int* slots, void* k_cache, void* v_cache, int n_tokens,
                         int q_heads, int kv_heads, int head_dim, pkv_stream stream) {
  return pkv::rope_append_impl<__nv_bfloat16>(q, k, v, positions, cos_table, sin_table, slots, k_cache, v_cache, n_tokens,
                                              q_heads, kv_heads, head_dim, stream);
}
int pkv_rope_append_f32(void* q, const void* k, const void* v, const int* positions, const float* cos_table,
                        const float* sin_table, const int* slots, void* k_cache, void* v_cache, int n_tokens,
                        int q_heads, int kv_heads, int head_dim, pkv_stream stream) {
  return pkv::rope_append_impl<float>(q, k, v, positions, cos_table, sin_table, slots, k_cache, v_cache, n_tokens, q_heads,
                                      kv_heads, head_dim, stream);
}
}
