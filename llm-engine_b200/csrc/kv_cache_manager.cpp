// Host KV block bookkeeping: pkv::KVCacheManager (include/pkv_kv_cache.hpp).
//
// Behavioural contract = llm-engine's src/kv_cache/block_allocator.cpp:8-142.
// The facts that make block ids, hashes and statistics come out identical:
//   * free blocks are handed out lowest id first, and a released unhashed block
//     is the next one handed out (a LIFO stack seeded n-1 .. 0)          (:12-13, :50)
//   * eviction takes the least recently RELEASED unowned hashed block      (:27-33)
//   * a block is published under its chained hash only once every slot of it has
//     been computed, only if the previous block of the chain is published, and
//     only if no other block already carries that hash                     (:54-64, :130-137)
//   * a prompt's capacity check does not count LRU-resident hits as room   (:97-101)
//   * blocks are released last to first                                    (:139-142)
#include <cassert>
#include <stdexcept>

#include "pkv_kv_cache.hpp"

namespace pkv {

namespace {
constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;

inline uint64_t finalize64(uint64_t z) {
  z += kGolden;
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z;
}
}  // namespace

uint64_t KVCacheManager::hash_block(uint64_t prev_hash, const int32_t* tokens, int n) {
  uint64_t h = prev_hash ^ kGolden;
  for (int i = 0; i < n; ++i) h = finalize64(h ^ static_cast<uint64_t>(static_cast<uint32_t>(tokens[i])));
  return h ? h : 1;  // 0 means "unhashed"
}

KVCacheManager::KVCacheManager(int num_blocks, int block_size, bool enable_prefix_caching)
    : num_blocks_(num_blocks), block_size_(block_size), prefix_caching_(enable_prefix_caching) {
  if (num_blocks <= 0 || block_size <= 0) throw std::invalid_argument("num_blocks and block_size must be > 0");
  const size_t n = static_cast<size_t>(num_blocks);
  refs_.assign(n, 0);
  content_hash_.assign(n, 0);
  lru_prev_.assign(n, kNoBlock);
  lru_next_.assign(n, kNoBlock);
  in_lru_.assign(n, 0);
  free_stack_.resize(n);
  for (size_t i = 0; i < n; ++i) free_stack_[i] = static_cast<BlockId>(n - 1 - i);
}

void KVCacheManager::lru_unlink(BlockId b) {
  if (!in_lru_[b]) return;
  const BlockId p = lru_prev_[b], nx = lru_next_[b];
  if (p == kNoBlock) lru_head_ = nx; else lru_next_[p] = nx;
  if (nx == kNoBlock) lru_tail_ = p; else lru_prev_[nx] = p;
  lru_prev_[b] = lru_next_[b] = kNoBlock;
  in_lru_[b] = 0;
  --lru_count_;
}

void KVCacheManager::lru_push_back(BlockId b) {
  lru_prev_[b] = lru_tail_;
  lru_next_[b] = kNoBlock;
  if (lru_tail_ == kNoBlock) lru_head_ = b; else lru_next_[lru_tail_] = b;
  lru_tail_ = b;
  in_lru_[b] = 1;
  ++lru_count_;
}

BlockId KVCacheManager::take_block() {
  if (!free_stack_.empty()) {
    const BlockId b = free_stack_.back();
    free_stack_.pop_back();
    return b;
  }
  if (lru_head_ == kNoBlock) return kNoBlock;
  const BlockId victim = lru_head_;
  lru_unlink(victim);
  published_.erase(content_hash_[victim]);
  content_hash_[victim] = 0;
  ++stats_.evictions;
  return victim;
}

void KVCacheManager::release_block(BlockId b, uint64_t hash) {
  assert(refs_[b] > 0);
  if (--refs_[b] > 0) return;
  const bool keep = prefix_caching_ && hash != 0 && content_hash_[b] == hash;
  if (keep) {
    lru_push_back(b);
    return;
  }
  if (content_hash_[b] != 0) {
    published_.erase(content_hash_[b]);
    content_hash_[b] = 0;
  }
  free_stack_.push_back(b);
}

void KVCacheManager::publish(BlockTable& bt, int idx, const int32_t* tokens) {
  if (!prefix_caching_) return;
  uint64_t chain = 0;
  if (idx > 0) {
    chain = bt.hashes[idx - 1];
    if (chain == 0) return;  // the chain broke earlier (a duplicate block); stay unhashed
  }
  const uint64_t h = hash_block(chain, tokens + static_cast<size_t>(idx) * block_size_, block_size_);
  if (!published_.emplace(h, bt.blocks[idx]).second) return;  // someone else already stands for this content
  content_hash_[bt.blocks[idx]] = h;
  bt.hashes[idx] = h;
}

int KVCacheManager::lookup_cached_prefix(const int32_t* tokens, int n) const {
  if (!prefix_caching_) return 0;
  const int full = n / block_size_;
  uint64_t chain = 0;
  int i = 0;
  for (; i < full; ++i) {
    chain = hash_block(chain, tokens + static_cast<size_t>(i) * block_size_, block_size_);
    if (published_.find(chain) == published_.end()) break;
  }
  return i * block_size_;
}

int KVCacheManager::lookup_cached_prefix(const std::vector<int32_t>& tokens) const {
  return lookup_cached_prefix(tokens.data(), static_cast<int>(tokens.size()));
}

std::optional<int> KVCacheManager::allocate_prompt(BlockTable& bt, const int32_t* tokens, int n) {
  assert(bt.empty());
  const int total = blocks_needed(n, block_size_);
  const int full = n / block_size_;
  ++stats_.prefix_queries;
  stats_.prefix_total_blocks += static_cast<uint64_t>(full);

  // Leading full blocks already published: reusing them costs no pool capacity,
  // unless they currently sit in the LRU, in which case they are part of
  // num_available_blocks() and must not be counted twice.
  int hit = 0, hit_in_lru = 0;
  if (prefix_caching_) {
    uint64_t chain = 0;
    bt.blocks.reserve(static_cast<size_t>(total));
    bt.hashes.reserve(static_cast<size_t>(total));
    for (; hit < full; ++hit) {
      chain = hash_block(chain, tokens + static_cast<size_t>(hit) * block_size_, block_size_);
      auto it = published_.find(chain);
      if (it == published_.end()) break;
      bt.blocks.push_back(it->second);
      bt.hashes.push_back(chain);
      if (refs_[it->second] == 0) ++hit_in_lru;
    }
  }
  if (total - hit > num_available_blocks() - hit_in_lru) {
    bt.blocks.clear();
    bt.hashes.clear();
    ++stats_.allocation_failures;
    return std::nullopt;
  }
  for (int i = 0; i < hit; ++i) {
    lru_unlink(bt.blocks[i]);
    ++refs_[bt.blocks[i]];
  }
  stats_.prefix_hit_blocks += static_cast<uint64_t>(hit);
  for (int i = hit; i < total; ++i) {
    const BlockId b = take_block();
    assert(b != kNoBlock);
    refs_[b] = 1;
    bt.blocks.push_back(b);
    bt.hashes.push_back(0);
  }
  bt.num_committed = hit;
  return hit * block_size_;
}

std::optional<int> KVCacheManager::allocate_prompt(BlockTable& bt, const std::vector<int32_t>& tokens) {
  return allocate_prompt(bt, tokens.data(), static_cast<int>(tokens.size()));
}

bool KVCacheManager::ensure_slot(BlockTable& bt, int num_tokens) {
  const int total = blocks_needed(num_tokens, block_size_);
  assert(total <= bt.num_blocks() + 1);
  if (total <= bt.num_blocks()) return true;
  const BlockId b = take_block();
  if (b == kNoBlock) {
    ++stats_.allocation_failures;
    return false;
  }
  refs_[b] = 1;
  bt.blocks.push_back(b);
  bt.hashes.push_back(0);
  return true;
}

void KVCacheManager::commit_computed(BlockTable& bt, const int32_t* tokens, int n, int num_computed) {
  if (!prefix_caching_) return;
  assert(num_computed <= n);
  (void)n;
  for (; bt.num_committed < bt.num_blocks() && (bt.num_committed + 1) * block_size_ <= num_computed;
       ++bt.num_committed)
    publish(bt, bt.num_committed, tokens);
}

void KVCacheManager::commit_computed(BlockTable& bt, const std::vector<int32_t>& tokens, int num_computed) {
  commit_computed(bt, tokens.data(), static_cast<int>(tokens.size()), num_computed);
}

void KVCacheManager::free(BlockTable& bt) {
  for (int i = bt.num_blocks(); i-- > 0;) release_block(bt.blocks[i], bt.hashes[i]);
  bt.blocks.clear();
  bt.hashes.clear();
  bt.num_committed = 0;
}

void KVCacheManager::fork(const BlockTable& parent, BlockTable& child) {
  assert(child.empty());
  child.blocks = parent.blocks;
  child.hashes = parent.hashes;
  child.num_committed = parent.num_committed;
  for (BlockId b : child.blocks) ++refs_[b];
}

std::optional<std::pair<BlockId, BlockId>> KVCacheManager::cow(BlockTable& bt, int write_pos) {
  const int idx = write_pos / block_size_;
  const std::pair<BlockId, BlockId> none{kNoBlock, kNoBlock};
  // Committed blocks are full and published; llm-engine only ever re-writes them
  // with identical values (src/scheduler/scheduler.cpp:60), so they are left shared.
  if (idx >= bt.num_blocks() || idx < bt.num_committed) return none;
  const BlockId src = bt.blocks[idx];
  if (refs_[src] <= 1) return none;
  const BlockId dst = take_block();
  if (dst == kNoBlock) {
    ++stats_.allocation_failures;
    return std::nullopt;
  }
  refs_[dst] = 1;
  --refs_[src];
  bt.blocks[idx] = dst;
  bt.hashes[idx] = 0;
  return std::make_pair(src, dst);
}

}  // namespace pkv
