// llm-engine's own launcher symbols, re-defined on top of the C ABI.
//
// include/engine/cuda_kernels.h of llm-engine declares (lines 43-62)
//     engine::launch_store_kv, engine::launch_attention_decode,
//     engine::launch_attention_decode_gqa
// and src/model/cuda/cuda_model.cu:368-377 calls them once per layer.  This file
// defines those three functions with exactly those signatures, so llm-engine
// links against libpkv instead of compiling src/kernels/store_kv.cu,
// attention_decode.cu and attention_decode_gqa.cu, with no change to its sources.
//
// Error behaviour follows the reference launchers: empty steps are silent no-ops,
// unsupported geometry throws std::runtime_error before anything is enqueued
// (src/kernels/attention_decode.cu:147-154, attention_decode_gqa.cu:211-224), and
// nothing here synchronises the device.
//
// Every packed token of a step comes through launch_attention_decode, prefill chunks
// included (src/model/cuda/cuda_model.cu:362-377).  The launchers hand the step to
// pkv_mixed_attn_f16, which finds the chunks on the device and sends them to the
// tensor-core prefill kernel and everything else to the decode kernels; geometries the
// prefill kernel does not run take the decode path, as before.
//
// The reference signatures carry no workspace argument, so split-K and router scratch
// is kept here in a grow-only device buffer per GPU -- the same pattern as the
// caller's own Scratch<T> buffers (src/model/cuda/cuda_model.cu:212-233).  A larger
// buffer is allocated when a step needs more than any step before it, which is the
// one moment this file calls cudaMalloc (so: not during stream capture, where
// allocation is illegal; size the first step generously or warm up before capturing).
// Buffers that were outgrown are kept until the process exits rather than freed: work
// already enqueued may still use them, and cudaFree would wait for the device.  One
// buffer per device serves every stream: calls on different streams of one device
// must not overlap, as with the caller's own single-stream scratch.  Set
// PKV_SHIM_NO_WORKSPACE=1 to run without scratch (no split-K, no prefill routing).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "pkv.h"

namespace {

struct DeviceScratch {
  void* ptr = nullptr;
  size_t bytes = 0;
  std::vector<void*> outgrown;
};
constexpr int kMaxDevices = 64;
DeviceScratch g_scratch[kMaxDevices];
std::mutex g_mu;

void* scratch_for(size_t need, size_t* have) {
  static const bool disabled = [] { const char* e = std::getenv("PKV_SHIM_NO_WORKSPACE"); return e && *e == '1'; }();
  *have = 0;
  if (disabled || need == 0) return nullptr;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceScratch& s = g_scratch[dev];
  if (s.bytes < need) {
    const size_t grown = need + need / 2;
    void* p = nullptr;
    if (cudaMalloc(&p, grown) != cudaSuccess) {
      cudaGetLastError();
      if (s.bytes == 0) return nullptr;   // no scratch at all: the unsplit path rather than a failed step
      *have = s.bytes;                    // keep using the smaller buffer: the call sizes its plan to it
      return s.ptr;
    }
    if (s.ptr) s.outgrown.push_back(s.ptr);
    s.ptr = p;
    s.bytes = grown;
  }
  *have = s.bytes;
  return s.ptr;
}

[[noreturn]] void raise(const char* fn, int status) {
  throw std::runtime_error(std::string(fn) + ": " + pkv_status_string(status) + ": " + pkv_last_error());
}

void decode(const char* fn, const __half* q, const __half* k_cache, const __half* v_cache, const int* block_tables,
            const int* table_offset, const int* token_seq, const int* token_pos, __half* out, int n_tokens,
            int q_heads, int kv_heads, int head_dim, int block_size, float scale, cudaStream_t stream) {
  if (n_tokens <= 0 || q_heads <= 0 || kv_heads <= 0) return;
  size_t have = 0;
  void* ws = scratch_for(pkv_mixed_attn_workspace_bytes(n_tokens, q_heads, kv_heads, head_dim), &have);
  int st = pkv_mixed_attn_f16(q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out, n_tokens,
                              q_heads, kv_heads, head_dim, block_size, /*num_blocks=*/0, scale, /*min_run=*/0, ws, have,
                              stream);
  if (st == PKV_E_WORKSPACE)   // an outgrown buffer that could not be replaced: still correct without the router
    st = pkv_decode_attn_f16(q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out, n_tokens,
                             q_heads, kv_heads, head_dim, block_size, scale, ws, have, stream);
  if (st != PKV_OK) raise(fn, st);
}

}  // namespace

namespace engine {

void launch_store_kv(const __half* k, const __half* v, const int* slots, __half* k_cache, __half* v_cache,
                     int n_tokens, int kv_dim, cudaStream_t stream) {
  const int st = pkv_append_f16(k, v, slots, k_cache, v_cache, n_tokens, kv_dim, stream);
  if (st != PKV_OK) raise("launch_store_kv", st);
}

void launch_attention_decode(const __half* q, const __half* k_cache, const __half* v_cache,
                             const int* block_tables, const int* table_offset, const int* token_seq,
                             const int* token_pos, __half* out, int n_tokens, int q_heads, int kv_heads,
                             int head_dim, int block_size, float scale, cudaStream_t stream) {
  decode("launch_attention_decode", q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out,
         n_tokens, q_heads, kv_heads, head_dim, block_size, scale, stream);
}

// llm-engine selects between the two names with ENGINE_ATTN=gqa
// (src/model/cuda/cuda_model.cu:554-557); here both reach the same kernel, which
// always shares K/V reads across the GQA group.
void launch_attention_decode_gqa(const __half* q, const __half* k_cache, const __half* v_cache,
                                 const int* block_tables, const int* table_offset, const int* token_seq,
                                 const int* token_pos, __half* out, int n_tokens, int q_heads, int kv_heads,
                                 int head_dim, int block_size, float scale, cudaStream_t stream) {
  decode("launch_attention_decode_gqa", q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out,
         n_tokens, q_heads, kv_heads, head_dim, block_size, scale, stream);
}

}  // namespace engine
