// Host half of the C ABI (include/pkv.h): status strings, KVCacheManager handles
// and step-index packing.  No CUDA in this file.
#include <cstring>
#include <new>
#include <unordered_map>

#include "pkv.h"
#include "pkv_kv_cache.hpp"
#include "status.hpp"

namespace pkv {
namespace {
thread_local char g_err[512] = {0};
}
int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
void clear_error() { g_err[0] = 0; }
}  // namespace pkv

struct pkv_kvmgr { pkv::KVCacheManager impl; };
struct pkv_table { pkv::BlockTable impl; };

extern "C" {

int pkv_abi_version(void) { return PKV_ABI_VERSION; }

const char* pkv_status_string(int status) {
  switch (status) {
    case PKV_OK: return "ok";
    case PKV_E_ARG: return "invalid argument";
    case PKV_E_UNSUPPORTED: return "unsupported geometry";
    case PKV_E_WORKSPACE: return "workspace missing or too small";
    case PKV_E_CUDA: return "CUDA runtime error";
    case PKV_E_NOMEM: return "block pool exhausted";
    case PKV_E_STATE: return "invalid state";
    default: return "unknown status";
  }
}

const char* pkv_last_error(void) { return pkv::g_err; }

// ---- a0: bookkeeping handles ---------------------------------------------
pkv_kvmgr* pkv_kvmgr_create(int num_blocks, int block_size, int enable_prefix_caching) {
  if (num_blocks <= 0 || block_size <= 0) {
    pkv::fail(PKV_E_ARG, "pkv_kvmgr_create: num_blocks (%d) and block_size (%d) must be > 0", num_blocks, block_size);
    return nullptr;
  }
  try {
    return new pkv_kvmgr{pkv::KVCacheManager(num_blocks, block_size, enable_prefix_caching != 0)};
  } catch (const std::exception& e) {
    pkv::fail(PKV_E_ARG, "pkv_kvmgr_create: %s", e.what());
    return nullptr;
  }
}
void pkv_kvmgr_destroy(pkv_kvmgr* m) { delete m; }
pkv_table* pkv_table_create(void) { return new (std::nothrow) pkv_table{}; }
void pkv_table_destroy(pkv_table* t) { delete t; }

int pkv_kvmgr_allocate_prompt(pkv_kvmgr* m, pkv_table* t, const int32_t* tokens, int n) {
  if (!m || !t || (n > 0 && !tokens) || n < 0) return pkv::fail(PKV_E_ARG, "pkv_kvmgr_allocate_prompt: null handle or tokens");
  if (!t->impl.empty()) return pkv::fail(PKV_E_STATE, "pkv_kvmgr_allocate_prompt: table already holds blocks");
  auto r = m->impl.allocate_prompt(t->impl, tokens, n);
  return r ? *r : -1;
}
int pkv_kvmgr_ensure_slot(pkv_kvmgr* m, pkv_table* t, int num_tokens) {
  if (!m || !t) return pkv::fail(PKV_E_ARG, "pkv_kvmgr_ensure_slot: null handle");
  if (pkv::KVCacheManager::blocks_needed(num_tokens, m->impl.block_size()) > t->impl.num_blocks() + 1)
    return pkv::fail(PKV_E_STATE, "pkv_kvmgr_ensure_slot: %d tokens need more than one new block", num_tokens);
  return m->impl.ensure_slot(t->impl, num_tokens) ? 1 : 0;
}
void pkv_kvmgr_commit_computed(pkv_kvmgr* m, pkv_table* t, const int32_t* tokens, int n, int num_computed) {
  if (!m || !t || !tokens || num_computed > n) return;
  m->impl.commit_computed(t->impl, tokens, n, num_computed);
}
void pkv_kvmgr_free(pkv_kvmgr* m, pkv_table* t) {
  if (m && t) m->impl.free(t->impl);
}
int pkv_kvmgr_lookup_cached_prefix(const pkv_kvmgr* m, const int32_t* tokens, int n) {
  if (!m || (n > 0 && !tokens)) return 0;
  return m->impl.lookup_cached_prefix(tokens, n);
}
uint64_t pkv_hash_block(uint64_t prev_hash, const int32_t* tokens, int n) {
  return pkv::KVCacheManager::hash_block(prev_hash, tokens, n);
}
int pkv_kvmgr_block_size(const pkv_kvmgr* m) { return m->impl.block_size(); }
int pkv_kvmgr_num_total_blocks(const pkv_kvmgr* m) { return m->impl.num_total_blocks(); }
int pkv_kvmgr_capacity_tokens(const pkv_kvmgr* m) { return m->impl.capacity_tokens(); }
int pkv_kvmgr_num_free_blocks(const pkv_kvmgr* m) { return m->impl.num_free_blocks(); }
int pkv_kvmgr_num_cached_blocks(const pkv_kvmgr* m) { return m->impl.num_cached_blocks(); }
int pkv_kvmgr_num_available_blocks(const pkv_kvmgr* m) { return m->impl.num_available_blocks(); }
int pkv_kvmgr_num_used_blocks(const pkv_kvmgr* m) { return m->impl.num_used_blocks(); }
void pkv_kvmgr_stats(const pkv_kvmgr* m, uint64_t out[5]) {
  const pkv::KVCacheStats& s = m->impl.stats();
  out[0] = s.prefix_queries;
  out[1] = s.prefix_hit_blocks;
  out[2] = s.prefix_total_blocks;
  out[3] = s.evictions;
  out[4] = s.allocation_failures;
}
int pkv_kvmgr_ref_count(const pkv_kvmgr* m, int block) {
  if (!m || block < 0 || block >= m->impl.num_total_blocks()) return -1;
  return m->impl.ref_count(block);
}

int pkv_table_num_blocks(const pkv_table* t) { return t->impl.num_blocks(); }
int pkv_table_num_committed(const pkv_table* t) { return t->impl.num_committed; }
const int32_t* pkv_table_blocks(const pkv_table* t) { return t->impl.blocks.data(); }
const uint64_t* pkv_table_hashes(const pkv_table* t) { return t->impl.hashes.data(); }
int64_t pkv_table_slot(const pkv_table* t, int pos, int block_size) {
  if (!t || block_size <= 0 || pos < 0 || pos / block_size >= t->impl.num_blocks()) return -1;
  return t->impl.slot(pos, block_size);
}

int pkv_kvmgr_fork(pkv_kvmgr* m, const pkv_table* parent, pkv_table* child) {
  if (!m || !parent || !child) return pkv::fail(PKV_E_ARG, "pkv_kvmgr_fork: null handle");
  if (!child->impl.empty()) return pkv::fail(PKV_E_STATE, "pkv_kvmgr_fork: child table already holds blocks");
  m->impl.fork(parent->impl, child->impl);
  return PKV_OK;
}
int pkv_kvmgr_cow(pkv_kvmgr* m, pkv_table* t, int write_pos, int* src, int* dst) {
  if (!m || !t || !src || !dst || write_pos < 0) return pkv::fail(PKV_E_ARG, "pkv_kvmgr_cow: null handle or negative position");
  auto r = m->impl.cow(t->impl, write_pos);
  if (!r) return pkv::fail(PKV_E_NOMEM, "pkv_kvmgr_cow: no block left for the private copy");
  *src = r->first;
  *dst = r->second;
  return r->first == pkv::kNoBlock ? 0 : 1;
}

// ---- a4: step-index packing -------------------------------------------------
// Same outputs as the loop of CudaModel::upload_step_indices
// (src/model/cuda/cuda_model.cu:453-473), but sequences are recognised through a
// hash map instead of a linear scan per token, so a step of N tokens over S
// sequences costs O(N + sum of table lengths) rather than O(N*S).
int pkv_step_pack(int n_tokens, const uint64_t* tok_seq_key, const int32_t* const* tok_blocks,
                  const int* tok_num_blocks, const int* tok_pos, int block_size, int* slots,
                  int* token_seq, int* tables, size_t tables_cap, int* table_offset,
                  size_t offsets_cap, int* n_seqs, int* n_table) {
  if (n_tokens < 0 || block_size <= 0) return pkv::fail(PKV_E_ARG, "pkv_step_pack: n_tokens %d, block_size %d", n_tokens, block_size);
  if (!n_seqs || !n_table) return pkv::fail(PKV_E_ARG, "pkv_step_pack: null count outputs");
  *n_seqs = 0;
  *n_table = 0;
  if (n_tokens == 0) return PKV_OK;
  if (!tok_seq_key || !tok_blocks || !tok_num_blocks || !tok_pos || !slots || !token_seq || !tables || !table_offset)
    return pkv::fail(PKV_E_ARG, "pkv_step_pack: null array");
  std::unordered_map<uint64_t, int> index_of;
  index_of.reserve(static_cast<size_t>(n_tokens) * 2);
  size_t used = 0;
  int seqs = 0;
  for (int i = 0; i < n_tokens; ++i) {
    const int32_t* blocks = tok_blocks[i];
    const int nb = tok_num_blocks[i];
    const int pos = tok_pos[i];
    if (!blocks || pos < 0 || pos / block_size >= nb)
      return pkv::fail(PKV_E_ARG, "pkv_step_pack: token %d at position %d lies beyond its %d-block table", i, pos, nb);
    auto ins = index_of.emplace(tok_seq_key[i], seqs);
    if (ins.second) {
      if (static_cast<size_t>(seqs) >= offsets_cap || used + static_cast<size_t>(nb) > tables_cap)
        return pkv::fail(PKV_E_WORKSPACE, "pkv_step_pack: output capacity too small (tables %zu, offsets %zu)", tables_cap, offsets_cap);
      table_offset[seqs] = static_cast<int>(used);
      std::memcpy(tables + used, blocks, sizeof(int32_t) * static_cast<size_t>(nb));
      used += static_cast<size_t>(nb);
      ++seqs;
    }
    token_seq[i] = ins.first->second;
    slots[i] = static_cast<int>(static_cast<int64_t>(blocks[pos / block_size]) * block_size + pos % block_size);
  }
  *n_seqs = seqs;
  *n_table = static_cast<int>(used);
  return PKV_OK;
}

}  // extern "C"
