// Test harness (not product code): calls the three KV-path launchers of llm-engine by their C++
// names, in the order its forward pass does for one layer (src/model/cuda/cuda_model.cu:366-377:
// store_kv, then attention over every packed token of the step), and turns what they throw into
// a return code, so that a ctypes test can drive them.  The declarations are those of
// include/engine/cuda_kernels.h:43-62 of llm-engine; the definitions come from libpkv.so.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <exception>

namespace engine {
void launch_store_kv(const __half* k, const __half* v, const int* slots, __half* k_cache, __half* v_cache, int n_tokens,
                     int kv_dim, cudaStream_t stream);
void launch_attention_decode(const __half* q, const __half* k_cache, const __half* v_cache, const int* block_tables,
                             const int* table_offset, const int* token_seq, const int* token_pos, __half* out,
                             int n_tokens, int q_heads, int kv_heads, int head_dim, int block_size, float scale,
                             cudaStream_t stream);
void launch_attention_decode_gqa(const __half* q, const __half* k_cache, const __half* v_cache, const int* block_tables,
                                 const int* table_offset, const int* token_seq, const int* token_pos, __half* out,
                                 int n_tokens, int q_heads, int kv_heads, int head_dim, int block_size, float scale,
                                 cudaStream_t stream);
}  // namespace engine

extern "C" int harness_layer(int use_gqa, int do_store, const void* q, const void* k, const void* v, const int* slots,
                             void* k_cache, void* v_cache, const int* block_tables, const int* table_offset,
                             const int* token_seq, const int* token_pos, void* out, int n_tokens, int q_heads,
                             int kv_heads, int head_dim, int block_size, float scale, void* stream, char* err,
                             int err_len) {
  auto h = [](const void* p) { return static_cast<const __half*>(p); };
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  try {
    if (do_store)
      engine::launch_store_kv(h(k), h(v), slots, static_cast<__half*>(k_cache), static_cast<__half*>(v_cache), n_tokens,
                              kv_heads * head_dim, s);
    if (use_gqa)
      engine::launch_attention_decode_gqa(h(q), h(k_cache), h(v_cache), block_tables, table_offset, token_seq, token_pos,
                                          static_cast<__half*>(out), n_tokens, q_heads, kv_heads, head_dim, block_size,
                                          scale, s);
    else
      engine::launch_attention_decode(h(q), h(k_cache), h(v_cache), block_tables, table_offset, token_seq, token_pos,
                                      static_cast<__half*>(out), n_tokens, q_heads, kv_heads, head_dim, block_size, scale,
                                      s);
    return 0;
  } catch (const std::exception& e) {
    if (err && err_len > 0) {
      std::strncpy(err, e.what(), static_cast<size_t>(err_len) - 1);
      err[err_len - 1] = 0;
    }
    return 1;
  }
}
