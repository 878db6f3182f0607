// pkv_kv_cache.hpp -- host-side KV block bookkeeping for the paged-KV path.
//
// Keeps the public surface and the observable behaviour (block ids handed out,
// hashes, reference counts, LRU eviction order, statistics) of llm-engine's
// BlockTable / KVCacheManager (include/engine/kv_cache.h:21-99,
// src/kv_cache/block_allocator.cpp:8-142), so code written against those classes
// compiles and behaves the same when `engine::` is aliased to `pkv::`
// (include/engine/kv_cache.h in this repository does exactly that).
//
// Internals differ from the reference: the LRU of unowned hashed blocks is an
// intrusive doubly-linked list threaded through two int arrays (O(1) unlink with
// no node allocation and no side map), and the per-block state lives in one
// struct-of-arrays so a pool of 64 Ki blocks stays within a few hundred KB.
//
// Two additive operations, fork() and cow(), give copy-on-write of a shared
// partial block; llm-engine itself never needs it because it shares full blocks
// only (docs/design.md:36).
#pragma once

#include <cstdint>
#include <optional>
#include <unordered_map>
#include <utility>
#include <vector>

namespace pkv {

using BlockId = int32_t;
constexpr BlockId kNoBlock = -1;

// include/engine/kv_cache.h:21-32
struct BlockTable {
  std::vector<BlockId> blocks;
  std::vector<uint64_t> hashes;  // parallel to blocks; 0 = not (yet) hashed
  int num_committed = 0;         // leading blocks whose hash publication was attempted

  int num_blocks() const { return static_cast<int>(blocks.size()); }
  bool empty() const { return blocks.empty(); }
  int64_t slot(int pos, int block_size) const {
    return static_cast<int64_t>(blocks[pos / block_size]) * block_size + pos % block_size;
  }
};

// include/engine/kv_cache.h:34-40
struct KVCacheStats {
  uint64_t prefix_queries = 0;
  uint64_t prefix_hit_blocks = 0;
  uint64_t prefix_total_blocks = 0;
  uint64_t evictions = 0;
  uint64_t allocation_failures = 0;
};

class KVCacheManager {
 public:
  // Throws std::invalid_argument unless both sizes are positive (block_allocator.cpp:11).
  KVCacheManager(int num_blocks, int block_size, bool enable_prefix_caching);

  int block_size() const { return block_size_; }
  int num_total_blocks() const { return num_blocks_; }
  int capacity_tokens() const { return num_blocks_ * block_size_; }
  int num_free_blocks() const { return static_cast<int>(free_stack_.size()); }
  int num_cached_blocks() const { return lru_count_; }
  int num_available_blocks() const { return num_free_blocks() + num_cached_blocks(); }
  int num_used_blocks() const { return num_blocks_ - num_available_blocks(); }
  bool prefix_caching_enabled() const { return prefix_caching_; }
  const KVCacheStats& stats() const { return stats_; }
  int ref_count(BlockId b) const { return refs_[static_cast<size_t>(b)]; }

  static int blocks_needed(int num_tokens, int block_size) { return (num_tokens + block_size - 1) / block_size; }

  // kv_cache.h:58-62 / block_allocator.cpp:78-116
  std::optional<int> allocate_prompt(BlockTable& bt, const std::vector<int32_t>& tokens);
  std::optional<int> allocate_prompt(BlockTable& bt, const int32_t* tokens, int n);
  // kv_cache.h:64-66 / block_allocator.cpp:118-128
  bool ensure_slot(BlockTable& bt, int num_tokens);
  // kv_cache.h:68-72 / block_allocator.cpp:130-137
  void commit_computed(BlockTable& bt, const std::vector<int32_t>& tokens, int num_computed);
  void commit_computed(BlockTable& bt, const int32_t* tokens, int n, int num_computed);
  // kv_cache.h:74-76 / block_allocator.cpp:139-142
  void free(BlockTable& bt);
  // kv_cache.h:78-79 / block_allocator.cpp:66-76
  int lookup_cached_prefix(const std::vector<int32_t>& tokens) const;
  int lookup_cached_prefix(const int32_t* tokens, int n) const;
  // kv_cache.h:81 / block_allocator.cpp:16-23
  static uint64_t hash_block(uint64_t prev_hash, const int32_t* tokens, int n);

  // ---- additive: copy-on-write of a shared, not yet committed block ----------
  // `child` (must be empty) comes to share every block of `parent`.
  void fork(const BlockTable& parent, BlockTable& child);
  // Call before writing position write_pos.  Returns {src, dst} when the block
  // holding that position was shared and `bt` has been moved to the private block
  // dst (the caller must copy src -> dst before the write); {kNoBlock, kNoBlock}
  // when no copy is needed; nullopt when the pool is exhausted.
  std::optional<std::pair<BlockId, BlockId>> cow(BlockTable& bt, int write_pos);

 private:
  BlockId take_block();  // kNoBlock when neither a free nor an evictable block exists
  void release_block(BlockId b, uint64_t hash);
  void lru_unlink(BlockId b);
  void lru_push_back(BlockId b);
  void publish(BlockTable& bt, int block_idx, const int32_t* tokens);

  int num_blocks_, block_size_;
  bool prefix_caching_;
  std::vector<BlockId> free_stack_;        // back() is handed out next; lowest ids first
  std::vector<int> refs_;                  // owners per physical block
  std::vector<uint64_t> content_hash_;     // per physical block, 0 if unpublished
  std::vector<BlockId> lru_prev_, lru_next_;  // intrusive list; kNoBlock-terminated
  std::vector<uint8_t> in_lru_;
  BlockId lru_head_ = kNoBlock, lru_tail_ = kNoBlock;  // head = least recently released
  int lru_count_ = 0;
  std::unordered_map<uint64_t, BlockId> published_;
  KVCacheStats stats_;
};

}  // namespace pkv
