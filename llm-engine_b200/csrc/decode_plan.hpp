// Split-K work list for paged decode attention: layout of the caller's workspace
// and the rule that picks the chunk size.  Shared by the host planner, the device
// planner kernel and the attention kernels, so all three agree by construction.
//
// A decode step is a ragged batch: token t attends L_t = token_pos[t] + 1 keys and
// L_t can differ by 64x inside one batch.  One thread block per (token, kv head)
// would leave the GPU waiting for the longest sequence, so each token's key range
// is cut into chunks of `chunk` keys; a work item is (token, first key, key count).
// Tokens that fit one chunk write their output directly; the others write one
// partial (running max, denominator, unnormalised accumulator) per chunk, and the
// thread block that finishes a token's last outstanding chunk merges them.
//
// Workspace layout (every region 256-byte aligned):
//   header | tok_split[n_tokens] | counters[n_tokens*kv_heads] | items[cap_items]
//          | part_ml[cap_parts*q_heads*2] | part_acc[cap_parts*q_heads*head_dim]
// The first four regions up to items[n_items] form the "plan image" that the host
// planner uploads in one copy.
#pragma once

#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define PKV_HD __host__ __device__
#else
#define PKV_HD
#endif

namespace pkv {

constexpr int kPlanMagic = 0x706b7631;  // "pkv1"
constexpr int kNumChunkCandidates = 9;  // 64, 128, ..., 16384 keys
constexpr int kMinChunk = 64;

struct PlanHeader {
  int magic;
  int n_items;
  int chunk;  // 0 = tokens are not split
  int n_tokens;
  int n_parts;
  int kv_heads;
  int pad[2];
};

struct WorkItem {
  int token;
  int kv_begin;
  int kv_len;
  int part;  // partial slot to write, or -1 to write the final output directly
};

// A unit of the shared-prefix planner: up to four tokens whose sequences have the same blocks
// over keys [kv_begin, kv_begin + kv_len); each token's partial goes to its own slot.  Stored
// behind the ordinary items in the same workspace region, three 16-byte slots each.
struct SharedItem {
  int kv_begin, kv_len, n_tok, pad;
  int token[4];
  int part[4];
};
static_assert(sizeof(SharedItem) == 3 * sizeof(WorkItem), "three item slots");
constexpr int kSharedTokens = 4;

struct TokSplit {
  int part_base;  // first partial slot of this token (valid when nsplits > 1)
  int nsplits;
};

struct WsLayout {
  size_t off_tok, off_cnt, off_items, off_ml, off_acc, total;
  int cap_extra;  // items beyond one per token that fit
  int cap_items, cap_parts;
};

PKV_HD inline size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

// Layout for a workspace that admits `extra` work items beyond one per token
// (and therefore at most 2*extra partial slots: a token that is split at all
// contributes at least two items for one item of excess).
PKV_HD inline WsLayout ws_layout(int n_tokens, int q_heads, int kv_heads, int head_dim, int extra) {
  WsLayout w;
  w.cap_extra = extra;
  w.cap_items = n_tokens + extra;
  w.cap_parts = 2 * extra;
  size_t o = align256(sizeof(PlanHeader));
  w.off_tok = o;
  o = align256(o + sizeof(TokSplit) * static_cast<size_t>(n_tokens));
  w.off_cnt = o;
  o = align256(o + sizeof(int) * static_cast<size_t>(n_tokens) * kv_heads);
  w.off_items = o;
  o = align256(o + sizeof(WorkItem) * static_cast<size_t>(w.cap_items));
  w.off_ml = o;
  o = align256(o + sizeof(float) * 2 * static_cast<size_t>(w.cap_parts) * q_heads);
  w.off_acc = o;
  o = align256(o + sizeof(float) * static_cast<size_t>(w.cap_parts) * q_heads * head_dim);
  w.total = o;
  return w;
}

// Largest `extra` whose layout fits in `bytes`, or -1 if not even extra = 0 fits.
inline int ws_extra_for_bytes(int n_tokens, int q_heads, int kv_heads, int head_dim, size_t bytes, int max_extra) {
  if (ws_layout(n_tokens, q_heads, kv_heads, head_dim, 0).total > bytes) return -1;
  int lo = 0, hi = max_extra;
  while (lo < hi) {
    const int mid = lo + (hi - lo + 1) / 2;
    if (ws_layout(n_tokens, q_heads, kv_heads, head_dim, mid).total <= bytes) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Chunk rule.  items_at[j] = sum over tokens of ceil(L_t / (64 << j)).
//   1. take the smallest chunk >= 256 keys whose item count stays within the
//      budget (one item per token plus `extra_budget`): the most parallelism the
//      workspace and the target grid allow, without paying a partial per 16 KB;
//   2. if that still leaves fewer units than the GPU has workers (warps), go down to
//      128 keys if the budget allows (64-key units were measured slower: the fixed
//      cost per unit outweighs the extra parallelism).
// Returns 0 when no candidate fits (tokens are then processed unsplit).
PKV_HD inline int choose_chunk(const long long* items_at, int n_tokens, int kv_heads, long long extra_budget,
                               int wave_ctas, int forced_chunk) {
  if (forced_chunk > 0) {
    for (int j = 0; j < kNumChunkCandidates; ++j)
      if ((kMinChunk << j) == forced_chunk && items_at[j] - n_tokens <= extra_budget) return forced_chunk;
  }
  int best = -1;
  for (int j = 2; j < kNumChunkCandidates; ++j) {
    if (items_at[j] - n_tokens <= extra_budget) { best = j; break; }
  }
  if (best < 0) return 0;
  if (best == 2 && items_at[best] * kv_heads < wave_ctas && items_at[1] - n_tokens <= extra_budget) best = 1;
  return kMinChunk << best;
}

}  // namespace pkv
