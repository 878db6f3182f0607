/*
 * TEST INFRASTRUCTURE -- NOT PRODUCT CODE.
 *
 * A plain-C, CPU-only restatement of llm-engine's paged-KV hot path, used as the
 * checker the CUDA kernels are compared against.  Nothing in the shipped library
 * links, loads or calls this file; only the test-suite, the smoke check and the
 * benchmark's cpu_baseline leg do.
 *
 * Parity status: PINNED.  Every function below is checked (tests/test_oracle.py)
 *   - against the known-answer values the reference's own unit tests hold
 *     (tests/test_tensor.cpp:7-33 for the casts, tests/test_block_allocator.cpp:39
 *     for slot()), and
 *   - against the reference's own code compiled from its sources
 *     (oracle/_ref/libpkv_ref.so, built by oracle/Makefile) on seeded inputs,
 *     where the two must agree bit for bit, and
 *   - against committed golden fixtures generated from that compiled reference
 *     (tests/golden/).
 *
 * Each function cites the reference file:line whose arithmetic it follows.
 * The order of floating-point operations is kept identical to the reference's so
 * that, compiled without -ffast-math, results match it exactly.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------- casts ---- */

/* include/engine/tensor.h:20-22 : widen bf16 by placing it in the high half. */
float orc_bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* include/engine/tensor.h:23-28 : round-to-nearest-even; inf/nan truncated. */
uint16_t orc_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)(u >> 16);
  uint32_t lsb = (u >> 16) & 1u;
  return (uint16_t)((u + 0x7fffu + lsb) >> 16);
}

/* include/engine/tensor.h:29-41 : fp16 -> fp32 incl. subnormals, inf, nan. */
float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      int e = 0;
      man <<= 1;
      while ((man & 0x400u) == 0) { man <<= 1; e++; }
      man &= 0x3ffu;
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* include/engine/tensor.h:42-62 : fp32 -> fp16, round-to-nearest-even, with
 * overflow to inf and gradual underflow. */
uint16_t orc_f32_to_f16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint32_t sign = (u >> 16) & 0x8000u;
  uint32_t bexp = (u >> 23) & 0xffu;
  int32_t exp = (int32_t)bexp - 127 + 15;
  uint32_t man = u & 0x7fffffu;
  if (bexp == 0xffu) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0u));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    uint32_t shift = (uint32_t)(14 - exp);
    uint32_t half = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t mid = 1u << (shift - 1u);
    if (rem > mid || (rem == mid && (half & 1u))) half++;
    return (uint16_t)(sign | half);
  }
  uint32_t half = sign | ((uint32_t)exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
  return (uint16_t)half;
}

void orc_f32_to_bf16_array(const float* in, uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = orc_f32_to_bf16(in[i]);
}
void orc_bf16_to_f32_array(const uint16_t* in, float* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = orc_bf16_to_f32(in[i]);
}
void orc_f32_to_f16_array(const float* in, uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = orc_f32_to_f16(in[i]);
}
void orc_f16_to_f32_array(const uint16_t* in, float* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = orc_f16_to_f32(in[i]);
}

/* ------------------------------------------------------- block tables ---- */

/* include/engine/kv_cache.h:29-31 : physical slot of logical position `pos`. */
int64_t orc_slot(const int32_t* blocks, int pos, int block_size) {
  return (int64_t)blocks[pos / block_size] * block_size + pos % block_size;
}

/* src/kv_cache/block_allocator.cpp:16-23 : chained splitmix64-style block hash;
 * 0 is reserved for "unhashed" and is remapped to 1. */
static uint64_t orc_mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
uint64_t orc_hash_block(uint64_t prev_hash, const int32_t* tokens, int n) {
  uint64_t h = prev_hash ^ 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < n; i++) h = orc_mix64(h ^ (uint64_t)(uint32_t)tokens[i]);
  return h == 0 ? 1 : h;
}

/* src/model/cuda/cuda_model.cu:453-473 : per-step index packing.  Sequences are
 * numbered in order of first appearance among the packed tokens; each distinct
 * sequence's block table is appended once to `tables`.  `tok_seq_key[i]`
 * identifies token i's sequence (the reference compares Sequence pointers);
 * `tok_blocks[i]` / `tok_num_blocks[i]` is that sequence's table.
 * Returns the number of distinct sequences; *n_table receives len(tables). */
int orc_step_pack(int n_tokens, const uint64_t* tok_seq_key, const int32_t* const* tok_blocks,
                  const int* tok_num_blocks, const int* tok_pos, int block_size, int* slots,
                  int* token_seq, int* tables, int* table_offset, int* n_table) {
  int n_seen = 0, nt = 0;
  uint64_t* seen = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(n_tokens > 0 ? n_tokens : 1));
  for (int i = 0; i < n_tokens; i++) {
    int idx = -1;
    for (int j = 0; j < n_seen; j++)
      if (seen[j] == tok_seq_key[i]) { idx = j; break; }
    if (idx < 0) {
      idx = n_seen;
      seen[n_seen++] = tok_seq_key[i];
      table_offset[idx] = nt;
      for (int b = 0; b < tok_num_blocks[i]; b++) tables[nt++] = tok_blocks[i][b];
    }
    token_seq[i] = idx;
    slots[i] = (int)orc_slot(tok_blocks[i], tok_pos[i], block_size);
  }
  free(seen);
  *n_table = nt;
  return n_seen;
}

/* -------------------------------------------------------------- rope ---- */

/* include/engine/ops.h:34-51 : cos/sin tables [max_positions][head_dim/2], angles in double. */
void orc_rope_tables(int head_dim, int max_positions, float theta, float* cos_out, float* sin_out) {
  const int half = head_dim / 2;
  for (int i = 0; i < half; i++) {
    const double inv_freq = 1.0 / pow((double)theta, (2.0 * i) / head_dim);
    for (int p = 0; p < max_positions; p++) {
      const double angle = p * inv_freq;
      cos_out[(size_t)p * half + i] = (float)cos(angle);
      sin_out[(size_t)p * half + i] = (float)sin(angle);
    }
  }
}

/* include/engine/ops.h:56-68 : rotate_half RoPE in place on `heads` consecutive heads of one token. */
void orc_rope_inplace(float* x, int heads, int head_dim, int pos, const float* cos_table, const float* sin_table) {
  const int half = head_dim / 2;
  const float* c = cos_table + (size_t)pos * half;
  const float* s = sin_table + (size_t)pos * half;
  for (int h = 0; h < heads; h++) {
    float* v = x + h * head_dim;
    for (int i = 0; i < half; i++) {
      const float a = v[i], b = v[i + half];
      v[i] = a * c[i] - b * s[i];
      v[i + half] = b * c[i] + a * s[i];
    }
  }
}

/* ------------------------------------------------------------ append ---- */

/* src/model/cpu/cpu_model.cpp:153-157 (CPU) and src/kernels/store_kv.cu:20-29
 * (CUDA): each token's K and V row is copied to row `slots[t]` of the pool.
 * `row_bytes` = kv_dim * element size; tokens are applied in order. */
void orc_append(const void* k, const void* v, const int* slots, void* k_cache, void* v_cache,
                int n_tokens, size_t row_bytes) {
  for (int t = 0; t < n_tokens; t++) {
    memcpy((char*)k_cache + (size_t)slots[t] * row_bytes, (const char*)k + (size_t)t * row_bytes, row_bytes);
    memcpy((char*)v_cache + (size_t)slots[t] * row_bytes, (const char*)v + (size_t)t * row_bytes, row_bytes);
  }
}

/* Block copy for copy-on-write.  The reference has no such function (it never
 * shares a partial block, docs/design.md:36); the semantics fixed here are those
 * of memcpy applied pair by pair, in order, to both pools. */
void orc_copy_blocks(void* k_cache, void* v_cache, const int* src_dst_pairs, int n_pairs,
                     size_t block_bytes) {
  for (int i = 0; i < n_pairs; i++) {
    size_t s = (size_t)src_dst_pairs[2 * i] * block_bytes, d = (size_t)src_dst_pairs[2 * i + 1] * block_bytes;
    memcpy((char*)k_cache + d, (const char*)k_cache + s, block_bytes);
    memcpy((char*)v_cache + d, (const char*)v_cache + s, block_bytes);
  }
}

/* --------------------------------------------------------- attention ---- */

/* include/engine/ops.h:87-111 : attention for one (token, head).  Three passes
 * over positions 0..pos inclusive: scores and their max; exp with a double
 * denominator; weighted sum of V.  `scratch` holds pos+1 floats. */
void orc_paged_attention_head(const float* q, const float* k_cache, const float* v_cache,
                              const int32_t* blocks, int block_size, int pos, int kv_head,
                              int kv_heads, int head_dim, float scale, float* out, float* scratch) {
  const int kv_dim = kv_heads * head_dim;
  float mx = -INFINITY;
  for (int p = 0; p <= pos; p++) {
    const float* k = k_cache + (size_t)orc_slot(blocks, p, block_size) * kv_dim + kv_head * head_dim;
    float s = 0.f;
    for (int d = 0; d < head_dim; d++) s += q[d] * k[d];
    s *= scale;
    scratch[p] = s;
    if (s > mx) mx = s;
  }
  double denom = 0;
  for (int p = 0; p <= pos; p++) {
    scratch[p] = expf(scratch[p] - mx);
    denom += scratch[p];
  }
  for (int d = 0; d < head_dim; d++) out[d] = 0.f;
  for (int p = 0; p <= pos; p++) {
    const float w = (float)(scratch[p] / denom);
    const float* v = v_cache + (size_t)orc_slot(blocks, p, block_size) * kv_dim + kv_head * head_dim;
    for (int d = 0; d < head_dim; d++) out[d] += w * v[d];
  }
}

typedef struct {
  const float *q, *kc, *vc;
  const int *block_tables, *table_offset, *token_seq, *token_pos;
  float* out;
  int q_heads, kv_heads, head_dim, block_size;
  float scale;
  int64_t begin, end;
} orc_attn_job;

/* src/model/cpu/cpu_model.cpp:173-182 : one work item per (token, head);
 * item w -> token w / q_heads, head w % q_heads, kv head = head / group. */
static void* orc_attn_range(void* arg) {
  orc_attn_job* j = (orc_attn_job*)arg;
  const int group = j->q_heads / j->kv_heads;
  const size_t H = (size_t)j->q_heads * j->head_dim;
  int cap = 0;
  float* scratch = NULL;
  for (int64_t w = j->begin; w < j->end; w++) {
    const int i = (int)(w / j->q_heads), h = (int)(w % j->q_heads);
    const int pos = j->token_pos[i];
    if (pos + 1 > cap) {
      cap = pos + 1;
      free(scratch);
      scratch = (float*)malloc(sizeof(float) * (size_t)cap);
    }
    orc_paged_attention_head(j->q + (size_t)i * H + (size_t)h * j->head_dim, j->kc, j->vc,
                             j->block_tables + j->table_offset[j->token_seq[i]], j->block_size, pos,
                             h / group, j->kv_heads, j->head_dim, j->scale,
                             j->out + (size_t)i * H + (size_t)h * j->head_dim, scratch);
  }
  free(scratch);
  return NULL;
}

/* The launcher-level operation (include/engine/cuda_kernels.h:48-53 argument
 * list, on host fp32 arrays).  With threads > 1 the (token, head) items are cut
 * into contiguous ranges of ceil(count/threads), as the reference's pool does
 * (include/engine/parallel.h:78-83); results do not depend on the split. */
void orc_paged_attention(const float* q, const float* k_cache, const float* v_cache,
                         const int* block_tables, const int* table_offset, const int* token_seq,
                         const int* token_pos, float* out, int n_tokens, int q_heads, int kv_heads,
                         int head_dim, int block_size, float scale, int threads) {
  if (n_tokens <= 0 || q_heads <= 0) return;
  const int64_t count = (int64_t)n_tokens * q_heads;
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  orc_attn_job jobs[256];
  pthread_t tid[256];
  const int64_t per = (count + threads - 1) / threads;
  int n = 0;
  for (int t = 0; t < threads; t++) {
    int64_t b = per * t, e = b + per < count ? b + per : count;
    if (b >= e) break;
    orc_attn_job j = {q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out,
                      q_heads, kv_heads, head_dim, block_size, scale, b, e};
    jobs[n++] = j;
  }
  for (int t = 1; t < n; t++) pthread_create(&tid[t], NULL, orc_attn_range, &jobs[t]);
  orc_attn_range(&jobs[0]);
  for (int t = 1; t < n; t++) pthread_join(tid[t], NULL);
}
