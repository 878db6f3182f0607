// TEST INFRASTRUCTURE -- NOT PRODUCT CODE.
//
// A C-ABI window onto llm-engine's own CPU implementation of the paged-KV path.
// This file contains no algorithm: it #includes the reference's headers where
// they lie (the include path is given by oracle/Makefile) and forwards to
//   engine::ref::paged_attention_head      include/engine/ops.h:87-111
//   engine::KVCacheManager / BlockTable    include/engine/kv_cache.h, src/kv_cache/block_allocator.cpp
//   engine::ThreadPool                     include/engine/parallel.h
//   engine::f32_to_bf16 & friends          include/engine/tensor.h:20-62
//   engine::Scheduler                      include/engine/scheduler.h, src/scheduler/scheduler.cpp
//                                          (only to GENERATE realistic steps: which slices a real
//                                          engine run puts into a step, with which block tables)
// so that the plain-C restatement in paged_oracle.c, and through it the CUDA
// kernels, can be compared with the real thing.  It is built into
// oracle/_ref/libpkv_ref.so, which is never linked into the shipped library.
#include <cstdint>
#include <cstring>
#include <vector>

#include "engine/kv_cache.h"
#include "engine/ops.h"
#include "engine/parallel.h"
#include "engine/scheduler.h"
#include "engine/tensor.h"

using engine::BlockTable;
using engine::KVCacheManager;

extern "C" {

float ref_bf16_to_f32(uint16_t h) { return engine::bf16_to_f32(h); }
uint16_t ref_f32_to_bf16(float f) { return engine::f32_to_bf16(f); }
float ref_f16_to_f32(uint16_t h) { return engine::f16_to_f32(h); }
uint16_t ref_f32_to_f16(float f) { return engine::f32_to_f16(f); }

void ref_f32_to_bf16_array(const float* in, uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = engine::f32_to_bf16(in[i]);
}
void ref_bf16_to_f32_array(const uint16_t* in, float* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = engine::bf16_to_f32(in[i]);
}
void ref_f32_to_f16_array(const float* in, uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = engine::f32_to_f16(in[i]);
}
void ref_f16_to_f32_array(const uint16_t* in, float* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = engine::f16_to_f32(in[i]);
}

int64_t ref_slot(const int32_t* blocks, int pos, int block_size) {
  BlockTable bt;
  bt.blocks.assign(blocks, blocks + pos / block_size + 1);
  return bt.slot(pos, block_size);
}

uint64_t ref_hash_block(uint64_t prev, const int32_t* tokens, int n) {
  return KVCacheManager::hash_block(prev, tokens, n);
}

int ref_default_thread_count() { return engine::default_thread_count(); }

// ---- KVCacheManager / BlockTable handles --------------------------------
void* ref_mgr_new(int num_blocks, int block_size, int prefix) {
  try { return new KVCacheManager(num_blocks, block_size, prefix != 0); } catch (...) { return nullptr; }
}
void ref_mgr_delete(void* m) { delete static_cast<KVCacheManager*>(m); }
void* ref_bt_new() { return new BlockTable(); }
void ref_bt_delete(void* b) { delete static_cast<BlockTable*>(b); }

int ref_mgr_allocate_prompt(void* m, void* b, const int32_t* tokens, int n) {
  std::vector<int32_t> t(tokens, tokens + n);
  auto r = static_cast<KVCacheManager*>(m)->allocate_prompt(*static_cast<BlockTable*>(b), t);
  return r.has_value() ? *r : -1;
}
int ref_mgr_ensure_slot(void* m, void* b, int num_tokens) {
  return static_cast<KVCacheManager*>(m)->ensure_slot(*static_cast<BlockTable*>(b), num_tokens) ? 1 : 0;
}
void ref_mgr_commit_computed(void* m, void* b, const int32_t* tokens, int n, int num_computed) {
  std::vector<int32_t> t(tokens, tokens + n);
  static_cast<KVCacheManager*>(m)->commit_computed(*static_cast<BlockTable*>(b), t, num_computed);
}
void ref_mgr_free(void* m, void* b) { static_cast<KVCacheManager*>(m)->free(*static_cast<BlockTable*>(b)); }
int ref_mgr_lookup_cached_prefix(void* m, const int32_t* tokens, int n) {
  std::vector<int32_t> t(tokens, tokens + n);
  return static_cast<KVCacheManager*>(m)->lookup_cached_prefix(t);
}
// what: 0 free, 1 cached, 2 available, 3 used, 4 total, 5 block_size, 6 capacity_tokens
int ref_mgr_count(void* m, int what) {
  auto* k = static_cast<KVCacheManager*>(m);
  switch (what) {
    case 0: return k->num_free_blocks();
    case 1: return k->num_cached_blocks();
    case 2: return k->num_available_blocks();
    case 3: return k->num_used_blocks();
    case 4: return k->num_total_blocks();
    case 5: return k->block_size();
    case 6: return k->capacity_tokens();
  }
  return -1;
}
// out[5]: prefix_queries, prefix_hit_blocks, prefix_total_blocks, evictions, allocation_failures
void ref_mgr_stats(void* m, uint64_t* out) {
  const auto& s = static_cast<KVCacheManager*>(m)->stats();
  out[0] = s.prefix_queries; out[1] = s.prefix_hit_blocks; out[2] = s.prefix_total_blocks;
  out[3] = s.evictions; out[4] = s.allocation_failures;
}
int ref_bt_num_blocks(void* b) { return static_cast<BlockTable*>(b)->num_blocks(); }
int ref_bt_num_committed(void* b) { return static_cast<BlockTable*>(b)->num_committed; }
void ref_bt_blocks(void* b, int32_t* out) {
  auto* t = static_cast<BlockTable*>(b);
  if (!t->blocks.empty()) std::memcpy(out, t->blocks.data(), t->blocks.size() * sizeof(int32_t));
}
void ref_bt_hashes(void* b, uint64_t* out) {
  auto* t = static_cast<BlockTable*>(b);
  if (!t->hashes.empty()) std::memcpy(out, t->hashes.data(), t->hashes.size() * sizeof(uint64_t));
}
int64_t ref_bt_slot(void* b, int pos, int block_size) { return static_cast<BlockTable*>(b)->slot(pos, block_size); }

// ---- RoPE (include/engine/ops.h:34-68) ------------------------------------
void ref_rope_tables(int head_dim, int max_positions, float theta, float* cos_out, float* sin_out) {
  engine::ref::RopeTables t;
  t.build(head_dim, max_positions, theta);
  std::memcpy(cos_out, t.cos.data(), t.cos.size() * sizeof(float));
  std::memcpy(sin_out, t.sin.data(), t.sin.size() * sizeof(float));
}
void ref_rope_inplace(float* x, int heads, int head_dim, int pos, const float* cos_table, const float* sin_table) {
  engine::ref::RopeTables t;
  t.half = head_dim / 2;
  const size_t n = static_cast<size_t>(pos + 1) * t.half;
  t.cos.assign(cos_table, cos_table + n);
  t.sin.assign(sin_table, sin_table + n);
  engine::ref::rope_inplace(x, heads, head_dim, pos, t);
}

// ---- the hot path on host fp32 arrays --------------------------------------
// K/V append: the reference does this inline with two memcpy calls per token
// (src/model/cpu/cpu_model.cpp:153-157); there is no function to call, so the
// same two calls are issued here on row_bytes-sized rows.
void ref_append(const void* k, const void* v, const int* slots, void* k_cache, void* v_cache,
                int n_tokens, size_t row_bytes) {
  for (int t = 0; t < n_tokens; t++) {
    std::memcpy(static_cast<char*>(k_cache) + static_cast<size_t>(slots[t]) * row_bytes,
                static_cast<const char*>(k) + static_cast<size_t>(t) * row_bytes, row_bytes);
    std::memcpy(static_cast<char*>(v_cache) + static_cast<size_t>(slots[t]) * row_bytes,
                static_cast<const char*>(v) + static_cast<size_t>(t) * row_bytes, row_bytes);
  }
}

// Attention for every packed (token, head), calling ref::paged_attention_head
// through engine::ThreadPool the way CpuModel::forward does
// (src/model/cpu/cpu_model.cpp:173-185), with the launcher's argument list
// (include/engine/cuda_kernels.h:48-53).
void ref_paged_attention(const float* q, const float* k_cache, const float* v_cache,
                         const int* block_tables, const int* table_offset, const int* token_seq,
                         const int* token_pos, float* out, int n_tokens, int q_heads, int kv_heads,
                         int head_dim, int block_size, float scale, int threads) {
  if (n_tokens <= 0 || q_heads <= 0) return;
  // Rebuild one BlockTable per step-local sequence from the concatenated tables.
  int n_seqs = 0;
  for (int i = 0; i < n_tokens; i++) n_seqs = token_seq[i] + 1 > n_seqs ? token_seq[i] + 1 : n_seqs;
  std::vector<int> need(n_seqs, 0);
  for (int i = 0; i < n_tokens; i++) {
    const int nb = token_pos[i] / block_size + 1;
    if (nb > need[token_seq[i]]) need[token_seq[i]] = nb;
  }
  std::vector<BlockTable> bts(n_seqs);
  for (int s = 0; s < n_seqs; s++)
    bts[s].blocks.assign(block_tables + table_offset[s], block_tables + table_offset[s] + need[s]);

  const int group = q_heads / kv_heads;
  const size_t H = static_cast<size_t>(q_heads) * head_dim;
  auto body = [&](int64_t begin, int64_t end) {
    std::vector<float> scores;
    for (int64_t w = begin; w < end; w++) {
      const int i = static_cast<int>(w / q_heads), h = static_cast<int>(w % q_heads);
      engine::ref::paged_attention_head(q + static_cast<size_t>(i) * H + static_cast<size_t>(h) * head_dim,
                                        k_cache, v_cache, bts[token_seq[i]], block_size, token_pos[i],
                                        h / group, kv_heads, head_dim, scale,
                                        out + static_cast<size_t>(i) * H + static_cast<size_t>(h) * head_dim,
                                        scores);
    }
  };
  engine::ThreadPool pool(threads);
  pool.parallel_for(static_cast<int64_t>(n_tokens) * q_heads, body);
}

// ---- the reference's scheduler as a generator of steps ------------------------------
// One KVCacheManager + Scheduler pair (include/engine/scheduler.h:60-75); requests are added with
// their prompt tokens, every ref_sched_step() is one Scheduler::schedule(), and ref_sched_done()
// is Scheduler::on_step_done() with the caller's "sampled" tokens.
struct RefSched {
  KVCacheManager kv;
  engine::Scheduler sched;
  std::vector<engine::SequencePtr> seqs;
  engine::StepInput step;
  RefSched(int nb, int bs, bool prefix, engine::SchedulerConfig cfg) : kv(nb, bs, prefix), sched(cfg, kv) {}
};

void* ref_sched_new(int num_blocks, int block_size, int prefix, int max_num_seqs, int max_batched_tokens, int chunk) {
  engine::SchedulerConfig cfg;
  cfg.max_num_seqs = max_num_seqs;
  cfg.max_num_batched_tokens = max_batched_tokens;
  cfg.prefill_chunk_size = chunk;
  try { return new RefSched(num_blocks, block_size, prefix != 0, cfg); } catch (...) { return nullptr; }
}
void ref_sched_delete(void* h) { delete static_cast<RefSched*>(h); }
// returns the sequence's id (its index in arrival order)
int ref_sched_add(void* h, const int32_t* prompt, int n, int max_tokens) {
  auto* r = static_cast<RefSched*>(h);
  auto s = std::make_shared<engine::Sequence>();
  s->id = r->seqs.size();
  s->tokens.assign(prompt, prompt + n);
  s->prompt_len = n;
  s->params.max_tokens = max_tokens;
  s->params.ignore_eos = true;
  r->seqs.push_back(s);
  r->sched.add(s);
  return static_cast<int>(s->id);
}
// One scheduling round.  Returns the number of slices (prefill slices first, then decode);
// slice i is (seq_id[i], start[i], len[i], needs_logits[i]).
int ref_sched_step(void* h, int* seq_id, int* start, int* len, int* needs_logits, int cap) {
  auto* r = static_cast<RefSched*>(h);
  r->step = r->sched.schedule();
  const int n = static_cast<int>(r->step.slices.size());
  for (int i = 0; i < n && i < cap; i++) {
    const auto& sl = r->step.slices[i];
    seq_id[i] = static_cast<int>(sl.seq->id);
    start[i] = sl.start;
    len[i] = sl.len;
    needs_logits[i] = sl.needs_logits ? 1 : 0;
  }
  return n;
}
int ref_sched_seq_blocks(void* h, int seq, int32_t* out, int cap) {
  auto* r = static_cast<RefSched*>(h);
  const auto& b = r->seqs[seq]->block_table.blocks;
  for (size_t i = 0; i < b.size() && static_cast<int>(i) < cap; i++) out[i] = b[i];
  return static_cast<int>(b.size());
}
int ref_sched_seq_tokens(void* h, int seq, int32_t* out, int cap) {
  auto* r = static_cast<RefSched*>(h);
  const auto& t = r->seqs[seq]->tokens;
  for (size_t i = 0; i < t.size() && static_cast<int>(i) < cap; i++) out[i] = t[i];
  return static_cast<int>(t.size());
}
void ref_sched_done(void* h, const int32_t* sampled, int n) {
  auto* r = static_cast<RefSched*>(h);
  r->sched.on_step_done(r->step, std::vector<int32_t>(sampled, sampled + n));
}
int ref_sched_has_work(void* h) { return static_cast<RefSched*>(h)->sched.has_work() ? 1 : 0; }
// out[4]: steps, preemptions, admitted, finished
void ref_sched_stats(void* h, uint64_t* out) {
  const auto& s = static_cast<RefSched*>(h)->sched.stats();
  out[0] = s.steps; out[1] = s.preemptions; out[2] = s.admitted; out[3] = s.finished;
}

}  // extern "C"
