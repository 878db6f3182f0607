// Paged (chunked) prefill attention on the 5th-generation tensor cores (sm_100a):
// entry points of include/pkv.h, "prefill attention".
//
// llm-engine has no prefill kernel (src/kernels/attention_prefill.cu:1 is a stub):
// every prompt token goes through the decode kernel and re-reads its whole history.
// Here a work item is 128 consecutive tokens of one sequence's chunk for one query
// head; its keys are walked in tiles of 64, so S = Q K^T and O = P V are dense
// 128 x 64 x 64 contractions issued as tcgen05.mma with the accumulators in tensor
// memory.  The result it must agree with is ref::paged_attention_head
// (include/engine/ops.h:87-111) applied to every (token, head) of the chunk.
//
// Thread blocks are persistent, two per SM: each takes items until none are left --
// from a ticket counter that belongs to the launch's stream, or, where no counter can
// be handed out safely (stream capture, more streams than counters), in a fixed
// serpentine deal of the length-ranked list -- and its roles run ahead of one another
// across items (the next
// item's Q and first K/V tiles are fetched, and its first scores computed, while the
// softmax warps still write the current item's output), which hides the 4,000-cycle
// start of an item (look-ups through the block table, first loads, first MMA) and the
// hand-over between blocks that a one-item-per-block grid pays every time.
//
// Roles inside a block of 192 threads:
//   warp 4 (one lane)   TMA producer: takes the ticket, publishes the item, loads its Q
//                       tile into one of two buffers, then per key tile four boxes of
//                       16 slots x 128 bytes for K and four for V, gathered through the
//                       block table into a four-stage ring (128-byte swizzle, which is
//                       also the canonical shared-memory layout of the MMA operands).
//   warp 5 (one lane)   MMA issuer: S[j] = Q K_j^T (4 MMAs of K=16) into one of two S
//                       buffers in tensor memory, then O += P_j V_j (4 MMAs of N = 80 whose A
//                       operand is read from tensor memory and whose last 16 columns give
//                       the row sums); tcgen05.commit signals the mbarriers.
//   warps 0-3           softmax: thread r owns row r (tensor-memory lane r).  The 64 scores
//                       of the row come to registers with tcgen05.ld, then row max, exp2,
//                       and P goes back with tcgen05.st as packed 16-bit pairs over the
//                       first 32 columns of the same S buffer; causal mask by absolute
//                       position, applied only on tiles that reach the diagonal.  O and the
//                       row sums (the product of P with a tile of ones) accumulate in tensor
//                       memory and are rescaled only when a row's maximum has grown by more
//                       than 2^8.
// S[j+1] is issued before P_j V_j, so the tensor core works on the next scores while
// the softmax warps are busy with the current ones; shared and tensor memory are
// sized so that two blocks share an SM and fill each other's bubbles.
//
// Every mbarrier wait is bounded: a wait that runs out sets bit 2 of the device error
// word and the block carries on to its tear-down (tensor memory is always released).
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "launch_util.hpp"
#include "status.hpp"
#include "tma_util.hpp"

namespace pkv {

__device__ unsigned int g_pkv_prefill_error = 0;

// Ticket and completion counters of the persistent kernel, one pair per (device, stream): launches
// on one stream never overlap between their first ticket and their last (stream order; a
// programmatically launched successor takes its first ticket only after griddepcontrol.wait), and
// the last block of a launch leaves its pair at zero.  Launches that cannot be tied to a stream
// that way (stream capture: the graph may be replayed anywhere; more live streams than pairs) use
// no counter at all: their blocks take items in a fixed order.
constexpr int kTicketSlots = 64;
__device__ unsigned int g_prefill_ticket[kTicketSlots];
__device__ unsigned int g_prefill_done[kTicketSlots];

namespace {

constexpr int kQTile = 128;     // query rows per block
constexpr int kKTile = 64;      // keys per tile
constexpr int kHd = 64;         // head_dim this kernel is written for
constexpr int kKVStages = 4;
constexpr int kBox = 16 * 128;                   // one TMA box: 16 slots x 128 bytes
constexpr int kQBytes = kQTile * 128;            // 128 rows x 128 bytes
constexpr int kKBytes = kKTile * 128;            // one K (or V, or P) tile: 64 keys x 128 bytes / 128 rows x 64 keys
constexpr int kSmemQ = 0;
constexpr int kSmemKV = kSmemQ + 2 * kQBytes;                // two Q tiles (this item's and the next), then kKVStages x (K, V)
constexpr int kSmemOnes = kSmemKV + kKVStages * 2 * kKBytes; // a V-shaped tile of 1.0: P x ones = row sums
constexpr int kSmemTotal = kSmemOnes + kKBytes + 1024;       // 105 KB: two blocks per SM
constexpr int kThreads = 192, kProducerWarp = 4, kMmaWarp = 5;   // warps 0-3: softmax, one thread per row of the tile
constexpr uint32_t kTmemCols = 256;                          // two blocks per SM share the 512 columns
constexpr uint32_t kTmemS = 0, kTmemO = 128, kTmemL = 192;   // S0 @0, S1 @64, O @128 (64) with the row sums right behind (16)
constexpr int kMaxRanked = 256;       // launches of up to this many (sequence, tile) groups hand them out longest first
constexpr float kRescaleThreshold = 8.f;                     // in log2 units: P stays below 2^8

struct PrefillArgs {
  const int* block_tables;
  const int* table_offset;
  const int* q_start;
  const int* q_len;
  const int* ctx_len;
  void* out;
  int q_heads, kv_heads, group;
  int block_size, bs_log2;
  float scale;
  // persistent scheduling: items = sequences x query-tile slots x heads, handed out by a ticket counter
  // (ticket == nullptr: dealt in a fixed order instead)
  unsigned int* ticket;
  unsigned int* done;
  int n_items, n_qtiles_max, n_seqs;
  // When non-null, { n_seqs, n_qtiles_max, n_items } are read from this device array instead (written
  // by an earlier kernel on the stream: the mixed-step router decides on the device which runs of
  // tokens are prefill chunks); the three fields above are then upper bounds that sized the grid.
  const int* dims;
  unsigned int* host_err;   // pinned host word that also receives a give-up (null: none)
};

// ---- tcgen05 wrappers -----------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// A operand in tensor memory (row i of A in lane i, two 16-bit elements per column).
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, rows of 128 bytes packed 8 to a
// 1024-byte group (stride-dimension offset 1024): the layout TMA writes and the
// canonical layout of both K-major operands (Q, K, P) and the MN-major one (V).
// `lbo_bytes` is the distance between successive 64-element column blocks of an MN-major
// operand (unused for the K-major operands, whose K extent per MMA stays inside one row).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes = 16) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>(1024u >> 4) << 32;     // stride-dimension offset: next group of 8 rows
  d |= static_cast<uint64_t>(1u) << 46;             // descriptor version of this architecture
  d |= static_cast<uint64_t>(2u) << 61;             // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16, fp32 accumulate, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(bool bf16, int n, bool b_mn_major) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Two fused multiply-adds in one instruction (packed fp32 pairs): (a0, a1) * (s, s) + (n, n).
__device__ __forceinline__ void ffma2(float a0, float a1, float s, float n, float& r0, float& r1) {
  asm("{\n .reg .b64 ra, rs, rn, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rs, {%4, %4};\n mov.b64 rn, {%5, %5};\n"
      " fma.rn.f32x2 rd, ra, rs, rn;\n mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(r0), "=f"(r1)
      : "f"(a0), "f"(a1), "f"(s), "f"(n));
}

// Three-input maximum: one instruction on this architecture.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ void give_up(unsigned int* host_err) {
  atomicOr(&g_pkv_prefill_error, 4u);
  if (host_err) {
    *reinterpret_cast<volatile unsigned int*>(host_err) = 4u;
    __threadfence_system();
  }
}

// What the TMA producer publishes about the work item it has fetched; the other roles read it
// from shared memory once the item's Q tile barrier has completed.
struct ItemDesc {
  int n_kt;        // key tiles; -1: no more items
  int head, row0, rows_here, kv_total, limit0;   // limit0 = last visible key position of row 0
  int pad[2];
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 2)
    prefill_tc_kernel(const PrefillArgs a, const __grid_constant__ CUtensorMap qmap,
                      const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr uint32_t kIdescQK = instr_desc(kBf16, kKTile, false);
  constexpr uint32_t kIdescPV = instr_desc(kBf16, kHd + 16, true);   // 64 output dims + 16 row-sum columns
  constexpr float kLog2e = 1.4426950408889634f;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bars[4 + 2 * kKVStages + 6];
  __shared__ __align__(16) ItemDesc s_item[2];
  __shared__ uint32_t tmem_base_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sQ = base + kSmemQ, sKV = base + kSmemKV, sOnes = base + kSmemOnes;
  const uint32_t bar0 = smem_u32(&bars[0]);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  enum { Q_FULL = 0, Q_EMPTY = 2, KV_FULL = 4, KV_EMPTY = KV_FULL + kKVStages, S_FULL = KV_EMPTY + kKVStages, P_FULL = S_FULL + 2, PV_DONE = P_FULL + 2 };

  // ---- on-chip set-up: touches no global memory, so it may overlap the previous launch ----
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(BAR(Q_FULL + i), 1);
      mbar_init(BAR(Q_EMPTY + i), 1 + 128);   // tcgen05.commit after the item's last Q K^T, and the softmax threads (one arrival of 32 per warp) once done with the item
    }
    for (int i = 0; i < kKVStages; ++i) {
      mbar_init(BAR(KV_FULL + i), 1);
      mbar_init(BAR(KV_EMPTY + i), 1);   // arrived by tcgen05.commit after P_j V_j
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(BAR(S_FULL + i), 1);     // tcgen05.commit after Q K_j^T
      mbar_init(BAR(P_FULL + i), 128);   // the softmax threads (one arrival of 32 per warp), after writing their rows of P_j
      mbar_init(BAR(PV_DONE + i), 1);    // tcgen05.commit after P_j V_j: O updated
    }
    mbar_fence_init();
  }
  if (threadIdx.x < kKTile) {
    // the tile of ones that makes columns 64..79 of every P V product the row sums of P
    const uint32_t one2 = pack2<T>(1.f, 1.f);
    unsigned char* orow = base_ptr + kSmemOnes + threadIdx.x * 128;
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(orow + ch * 16) = make_uint4(one2, one2, one2, one2);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;

  pdl_launch_dependents();
  pdl_wait();

  // Order in which the (sequence, query tile) groups are handed out: longest key range first, so that
  // the launch ends on its shortest items and the blocks finish together (with the natural order the
  // last blocks ran up to a tenth of the launch alone).  Every block ranks the groups itself, once:
  // a few hundred comparisons per thread for up to kMaxRanked groups; larger launches keep the
  // natural order, whose tail matters less the more items there are.
  __shared__ int s_key[kMaxRanked];
  __shared__ short s_order[kMaxRanked];
  const int n_seqs = a.dims ? __ldcg(a.dims) : a.n_seqs;
  const int n_qtiles_max = a.dims ? __ldcg(a.dims + 1) : a.n_qtiles_max;
  const int n_items = a.dims ? __ldcg(a.dims + 2) : a.n_items;
  const int n_groups = n_seqs * n_qtiles_max;
  const bool ranked = n_groups <= kMaxRanked;
  if (ranked) {
    for (int j = threadIdx.x; j < n_groups; j += kThreads) {
      const int z = j / n_qtiles_max, y = j - z * n_qtiles_max;
      const int ql = __ldg(a.q_len + z);
      const int nt = (ql + kQTile - 1) / kQTile;
      s_key[j] = y < nt ? __ldg(a.ctx_len + z) + min((nt - y) * kQTile, ql) : -1;   // keys that tile sees; -1: no such tile
    }
    __syncthreads();
    for (int j = threadIdx.x; j < n_groups; j += kThreads) {
      const int kj = s_key[j];
      int rank = 0;
      for (int k = 0; k < n_groups; ++k) {
        const int kk = s_key[k];
        rank += (kk > kj || (kk == kj && k < j)) ? 1 : 0;
      }
      s_order[rank] = static_cast<short>(j);
    }
    __syncthreads();
  }

  // The block is persistent: it takes (sequence, query tile, head) items until none are left.  Every
  // role runs its own loop over the items and keeps its own running counts of items (n) and key tiles
  // (g), from which ring stages, buffers and barrier parities follow; the roles are coupled only
  // through the barriers, so the producer prefetches the next item's Q and first K/V tiles, and the
  // MMA thread computes its first scores, while the softmax warps are still writing the current
  // item's output.
  // After one of this thread's waits has run out no further wait of its spins: the block falls
  // through its schedule and releases its tensor memory.  (The record of a give-up does not stop
  // later launches: each launch stands on its own.)
  bool dead = false;
  auto WAIT = [&](uint32_t bar, uint32_t parity) {
    if (dead) return;
    if (!mbar_wait(bar, parity)) {
      dead = true;
      give_up(a.host_err);
    }
  };

  if (warp == kProducerWarp) {
    // ================================ TMA producer ================================
    int n = 0, g = 0;
    unsigned round = 0;                                        // fixed deal: items taken so far
    for (;;) {
      dead = __shfl_sync(0xffffffffu, dead ? 1 : 0, 0) != 0;   // only lane 0 waits: keep the warp in step
      // next item that has work: heads fastest (the heads of a group share their K/V tiles through
      // L2), groups in the order ranked above (or: a sequence's query tiles from the longest key
      // range down, then sequences)
      ItemDesc d;
      int seq = 0;
      d.n_kt = -1;
      while (!dead) {
        unsigned t = 0;
        if (a.ticket != nullptr) {
          if (lane == 0) t = atomicAdd(a.ticket, 1u);
          t = __shfl_sync(0xffffffffu, t, 0);
        } else {
          // serpentine deal of the (length-ranked) list: block b takes place b of every even round and
          // place G - 1 - b of every odd one, so that no block collects the longest item of every round
          t = round * gridDim.x + ((round & 1u) ? gridDim.x - 1u - blockIdx.x : blockIdx.x);
          ++round;
        }
        if (t >= static_cast<unsigned>(n_items)) break;
        const int head = static_cast<int>(t % a.q_heads);
        int rest = static_cast<int>(t / a.q_heads);
        if (ranked) rest = s_order[rest];
        const int slot_y = rest % n_qtiles_max;
        seq = rest / n_qtiles_max;
        const int q_len = __ldg(a.q_len + seq);
        const int tile = (q_len + kQTile - 1) / kQTile - 1 - slot_y;
        if (tile < 0) continue;
        const int ctx = __ldg(a.ctx_len + seq);
        d.head = head;
        d.row0 = __ldg(a.q_start + seq) + tile * kQTile;
        d.rows_here = min(kQTile, q_len - tile * kQTile);
        d.kv_total = ctx + tile * kQTile + d.rows_here;
        d.limit0 = ctx + tile * kQTile;
        d.n_kt = (d.kv_total + kKTile - 1) / kKTile;
        break;
      }
      const int qb = n & 1;
      if (lane == 0) {
        WAIT(BAR(Q_EMPTY + qb), ((n >> 1) & 1) ^ 1);
        s_item[qb] = d;
        if (d.n_kt > 0 && !dead) {
          mbar_arrive_expect_tx(BAR(Q_FULL + qb), kQBytes);
          tma_load_2d(sQ + qb * kQBytes, &qmap, d.head * kHd, d.row0, BAR(Q_FULL + qb));
        } else {
          s_item[qb].n_kt = -1;
          mbar_arrive(BAR(Q_FULL + qb));        // "no more items"
        }
      }
      dead = __shfl_sync(0xffffffffu, dead ? 1 : 0, 0) != 0;
      if (d.n_kt <= 0 || dead) break;
      const int kvh = d.head / a.group;
      const int* tbl = a.block_tables + __ldg(a.table_offset + seq);
      for (int j = 0; j < d.n_kt; ++j, ++g) {
        const int st = g % kKVStages;
        const int rel = j * kKTile + (lane & 3) * 16;
        int ent = 0;
        if (rel < d.kv_total) ent = __ldg(tbl + (rel >> a.bs_log2));
        int y[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int e = __shfl_sync(0xffffffffu, ent, b);
          y[b] = (e << a.bs_log2) + ((j * kKTile + 16 * b) & (a.block_size - 1));
        }
        if (lane == 0) {
          WAIT(BAR(KV_EMPTY + st), ((g / kKVStages) & 1) ^ 1);
          int nvalid = 0;
#pragma unroll
          for (int b = 0; b < 4; ++b) nvalid += (j * kKTile + 16 * b < d.kv_total) ? 1 : 0;
          mbar_arrive_expect_tx(BAR(KV_FULL + st), static_cast<uint32_t>(nvalid) * 2u * kBox);
          const uint32_t kdst = sKV + st * 2 * kKBytes, vdst = kdst + kKBytes;
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            if (j * kKTile + 16 * b < d.kv_total) {
              tma_load_2d(kdst + b * kBox, &kmap, kvh * kHd, y[b], BAR(KV_FULL + st));
              tma_load_2d(vdst + b * kBox, &vmap, kvh * kHd, y[b], BAR(KV_FULL + st));
            }
          }
        }
        __syncwarp();
      }
      ++n;
    }
  } else if (warp == kMmaWarp) {
    // ================================ MMA issuer ================================
    // One thread issues everything.  A tcgen05.mma returns to the issuing thread at the rate the
    // tensor pipe retires them (48 cycles for 128 x 64 x 16 from shared memory, 45 with A in tensor
    // memory), a blocking try_wait costs a few hundred cycles even on a completed phase (mbar_wait
    // looks first), and the scalar code of a lone thread runs at one dependent instruction every
    // few cycles, so the schedule is kept to two waits, eight MMAs and three commits per key tile:
    //  * no separate "S buffer free" barrier: a softmax thread has read S_{g-1} and written P_{g-1}
    //    over it before it arrives on P_FULL_{g-1}; this thread waits for that, issues P_{g-1} V_{g-1},
    //    and only then S_{g+1} into the same buffer (instructions of one thread execute in order);
    //  * O += P V and the row sums of P come out of ONE MMA of N = 80: the B operand is MN-major,
    //    its first 64 columns are the V tile and its next column block, one leading-dimension
    //    offset away, is a tile of ones.
    // It does not wait for the softmax warps' epilogue: after an item's last P V it goes on to the
    // next item's first scores.
    if (lane == 0) {
      const uint64_t desc_q0 = smem_desc(sQ), desc_k0 = smem_desc(sKV);
      int n = 0, g = 0;
      while (!dead) {
        const int qb = n & 1;
        WAIT(BAR(Q_FULL + qb), (n >> 1) & 1);
        const int n_kt = s_item[qb].n_kt;
        if (n_kt <= 0 || dead) break;
        const uint64_t desc_q = desc_q0 + ((qb * kQBytes) >> 4);
        auto issue_qk = [&](int gg, bool last_of_item) {
          const int st = gg % kKVStages, sb = gg & 1;
          WAIT(BAR(KV_FULL + st), (gg / kKVStages) & 1);
          tc_fence_after();
          // descriptors differ only in their 14-bit start-address field: add to the low word
          const uint64_t kd = desc_k0 + ((st * 2 * kKBytes) >> 4);
#pragma unroll
          for (int ks = 0; ks < kHd / 16; ++ks)
            tc_mma(tmem + kTmemS + sb * 64, desc_q + 2 * ks, kd + 2 * ks, kIdescQK, ks > 0);
          tc_commit(BAR(S_FULL + sb));
          if (last_of_item) tc_commit(BAR(Q_EMPTY + qb));      // the Q tile has been read for the last time
        };
        issue_qk(g, n_kt == 1);
        for (int j = 0; j < n_kt; ++j, ++g) {
          const int st = g % kKVStages, sb = g & 1;
          if (j + 1 < n_kt) issue_qk(g + 1, j + 2 == n_kt);
          WAIT(BAR(P_FULL + sb), (g >> 1) & 1);
          tc_fence_after();
          const uint32_t v_base = sKV + st * 2 * kKBytes + kKBytes;
          const uint64_t vd = smem_desc(v_base, sOnes - v_base);
          const uint32_t p_addr = tmem + kTmemS + sb * 64;      // P lies over the first 32 columns of its S buffer
#pragma unroll
          for (int kk = 0; kk < kKTile / 16; ++kk)
            tc_mma_ts(tmem + kTmemO, p_addr + kk * 8, vd + kk * (kBox >> 4), kIdescPV, (j | kk) != 0);
          tc_commit(BAR(KV_EMPTY + st));
          tc_commit(BAR(PV_DONE + sb));
        }
        ++n;
      }
    }
    __syncwarp();
  } else {
    // ================================ softmax warps ================================
    const int r = threadIdx.x;                      // row of the tile == tensor-memory lane
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const float sl2 = a.scale * kLog2e;
    int n = 0, g = 0;
    while (!dead) {
      const int qb = n & 1;
      WAIT(BAR(Q_FULL + qb), (n >> 1) & 1);
      const ItemDesc d = s_item[qb];
      if (d.n_kt <= 0 || dead) break;
      const int n_kt = d.n_kt, kv_total = d.kv_total, rows_here = d.rows_here;
      const int limit = d.limit0 + min(r, rows_here - 1);   // last visible key position of this row
      // Reference maximum of the row.  It follows the true running maximum lazily: O and the row
      // sum stay in tensor memory and are only rescaled when the maximum has grown by more than
      // 2^8, so most tiles cost no read-modify-write of the accumulator at all.
      float m_used = -INFINITY;

      for (int j = 0; j < n_kt; ++j, ++g) {
        const int sb = g & 1;
        const int k0 = j * kKTile;
        WAIT(BAR(S_FULL + sb), (g >> 1) & 1);
        tc_fence_after();
        float sc[kKTile];
        {
          uint32_t v0[32], v1[32];
          tc_ld32(tmem + lane_addr + kTmemS + sb * 64, v0);
          tc_ld32(tmem + lane_addr + kTmemS + sb * 64 + 32, v1);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            sc[i] = __uint_as_float(v0[i]);
            sc[32 + i] = __uint_as_float(v1[i]);
          }
        }
        // Causal mask, only on tiles that reach past some row's last visible key (warp-uniform test).
        if (__any_sync(0xffffffffu, k0 + kKTile - 1 > limit)) {
#pragma unroll
          for (int i = 0; i < kKTile; ++i)
            if (k0 + i > limit) sc[i] = -INFINITY;
        }
        // Row maximum: eight independent chains of three-input maxima, two scores a step.
        float mx8[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) mx8[u] = fmaxf(sc[u], sc[8 + u]);
#pragma unroll
        for (int i = 16; i < kKTile; i += 16)
#pragma unroll
          for (int u = 0; u < 8; ++u) mx8[u] = max3(mx8[u], sc[i + u], sc[i + 8 + u]);
        const float mx = fmaxf(max3(mx8[0], mx8[1], mx8[2]), fmaxf(max3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
        if (j == 0) {
          m_used = mx;                                 // finite: key 0 is visible to every row
        } else if (__any_sync(0xffffffffu, (mx - m_used) * sl2 > kRescaleThreshold)) {
          // Rare: bring this warp's rows of O and of the row sums to the new maximum.  Each thread
          // owns its own tensor-memory lane; the previous tile's P V must have landed and this tile's
          // cannot start before this thread has arrived on P_FULL below.
          WAIT(BAR(PV_DONE + ((g - 1) & 1)), ((g - 1) >> 1) & 1);
          tc_fence_after();
          const float m_new = fmaxf(m_used, mx);
          const float f = ex2_approx((m_used - m_new) * sl2);
          m_used = m_new;
#pragma unroll
          for (int blk = 0; blk < 3; ++blk) {          // O: columns 128..191, row sums: 192..223
            uint32_t v[32];
            tc_ld32(tmem + lane_addr + kTmemO + blk * 32, v);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
            tc_st32(tmem + lane_addr + kTmemO + blk * 32, v);
          }
        }
        const float neg = -m_used * sl2;
        // P goes back into tensor memory as packed 16-bit pairs over the first 32 columns of the S
        // buffer it came from: this thread has all of its own row in registers, and the MMA thread
        // overwrites the buffer with the scores after next only after it has issued this P V.
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float x0, x1;
            ffma2(sc[c * 32 + 2 * i], sc[c * 32 + 2 * i + 1], sl2, neg, x0, x1);
            pk[i] = pack2<T>(ex2_approx(x0), ex2_approx(x1));
          }
          tc_st16(tmem + lane_addr + kTmemS + sb * 64 + c * 16, pk);
        }
        if (j == n_kt - 1 && kv_total - k0 < kKTile) {
          // Keys past the end of the sequence in the last tile: their P is zero, but the V rows
          // behind them are whatever the pool or the ring held; clear them so 0 * x stays 0.
          const int st = g % kKVStages;
          WAIT(BAR(KV_FULL + st), (g / kKVStages) & 1);
          if (r < kKTile && r >= kv_total - k0) {
            unsigned char* vrow = base_ptr + kSmemKV + st * 2 * kKBytes + kKBytes + r * 128;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(vrow + ch * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the cleared rows before the MMA reads them
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_warp(BAR(P_FULL + sb));
      }
      // epilogue: O / row sum.  The next item's first P V cannot overwrite O before this thread has
      // arrived on that tile's P_FULL, which it does after the loads below.
      WAIT(BAR(PV_DONE + ((g - 1) & 1)), ((g - 1) >> 1) & 1);
      tc_fence_after();
      {
        uint32_t o0[32], o1[32], lv[32];
        tc_ld32(tmem + lane_addr + kTmemO, o0);
        tc_ld32(tmem + lane_addr + kTmemO + 32, o1);
        tc_ld32(tmem + lane_addr + kTmemL, lv);
        tc_wait_ld();
        tc_fence_before();
        // The row goes through shared memory so that the global stores are whole 128-byte lines
        // (eight lanes per row) instead of 32 scattered 16-byte pieces per instruction.  The staging
        // area is the item's own Q tile, which nothing reads any more (the item's last Q K^T has
        // completed); each warp stages and drains its own 32 rows, 16-byte pieces XOR-swizzled
        // against bank conflicts.
        const float inv = 1.f / __uint_as_float(lv[0]);
        unsigned char* stage = base_ptr + kSmemQ + qb * kQBytes;
        unsigned char* my_row = stage + r * 128;
#pragma unroll
        for (int dd = 0; dd < 32; dd += 8) {
          uint4 w0, w1;
          w0.x = pack2<T>(__uint_as_float(o0[dd]) * inv, __uint_as_float(o0[dd + 1]) * inv);
          w0.y = pack2<T>(__uint_as_float(o0[dd + 2]) * inv, __uint_as_float(o0[dd + 3]) * inv);
          w0.z = pack2<T>(__uint_as_float(o0[dd + 4]) * inv, __uint_as_float(o0[dd + 5]) * inv);
          w0.w = pack2<T>(__uint_as_float(o0[dd + 6]) * inv, __uint_as_float(o0[dd + 7]) * inv);
          w1.x = pack2<T>(__uint_as_float(o1[dd]) * inv, __uint_as_float(o1[dd + 1]) * inv);
          w1.y = pack2<T>(__uint_as_float(o1[dd + 2]) * inv, __uint_as_float(o1[dd + 3]) * inv);
          w1.z = pack2<T>(__uint_as_float(o1[dd + 4]) * inv, __uint_as_float(o1[dd + 5]) * inv);
          w1.w = pack2<T>(__uint_as_float(o1[dd + 6]) * inv, __uint_as_float(o1[dd + 7]) * inv);
          *reinterpret_cast<uint4*>(my_row + ((((dd >> 3)) ^ (r & 7)) << 4)) = w0;
          *reinterpret_cast<uint4*>(my_row + ((((dd >> 3) + 4) ^ (r & 7)) << 4)) = w1;
        }
        __syncwarp();
        T* obase = static_cast<T*>(a.out) + (static_cast<size_t>(d.row0) * a.q_heads + d.head) * kHd;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = warp * 32 + i * 4 + (lane >> 3), ch = lane & 7;
          const uint4 w = *reinterpret_cast<const uint4*>(stage + row * 128 + ((ch ^ (row & 7)) << 4));
          if (row < rows_here)
            *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(obase + static_cast<size_t>(row) * a.q_heads * kHd) + ch * 16) = w;
        }
      }
      // The Q buffer may be refilled (by TMA) once every thread is done with it: the item's
      // description, and the staging of its output.
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_warp(BAR(Q_EMPTY + qb));
      ++n;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  // The last block out resets the ticket counter for the next launch on this stream.
  if (threadIdx.x == 0 && a.ticket != nullptr) {
    __threadfence();
    if (atomicAdd(a.done, 1u) == gridDim.x - 1) {
      *a.ticket = 0u;
      *a.done = 0u;
      __threadfence();
    }
  }
}

int log2_exact(int x) {
  if (x <= 0 || (x & (x - 1))) return -1;
  int l = 0;
  while ((1 << l) < x) ++l;
  return l;
}

// The ticket pair of (current device, stream), or null when none can be handed out safely: the
// stream is capturing (the graph could be replayed on any stream, next to anything), the table of
// pairs is full, or PKV_PREFILL_SCHED=static asks for the fixed deal.
struct TicketPair { unsigned int* ticket; unsigned int* done; };
TicketPair ticket_pair_for(cudaStream_t stream, int dev) {
  static const bool force_static = [] { const char* e = std::getenv("PKV_PREFILL_SCHED"); return e && e[0] == 's'; }();
  TicketPair none{nullptr, nullptr};
  if (force_static || dev < 0 || dev >= 64) return none;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) { cudaGetLastError(); return none; }
  if (cap != cudaStreamCaptureStatusNone) return none;
  struct PerDevice {
    unsigned int* ticket_base = nullptr;
    unsigned int* done_base = nullptr;
    cudaStream_t streams[kTicketSlots];
    int n = 0;
  };
  static PerDevice table[64];
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  PerDevice& d = table[dev];
  if (!d.ticket_base) {
    void *t = nullptr, *dn = nullptr;
    if (cudaGetSymbolAddress(&t, g_prefill_ticket) != cudaSuccess || cudaGetSymbolAddress(&dn, g_prefill_done) != cudaSuccess) {
      cudaGetLastError();
      return none;
    }
    d.ticket_base = static_cast<unsigned int*>(t);
    d.done_base = static_cast<unsigned int*>(dn);
  }
  int slot = -1;
  for (int i = 0; i < d.n; ++i)
    if (d.streams[i] == stream) { slot = i; break; }
  if (slot < 0) {
    if (d.n >= kTicketSlots) return none;
    slot = d.n++;
    d.streams[slot] = stream;
  }
  return TicketPair{d.ticket_base + slot, d.done_base + slot};
}

}  // namespace

unsigned int* error_mirror(bool create);                 // error_mirror.cu
int check_error_mirror(const char* fn);

// Shared by the C entry points below and by the mixed-step router (decode_attn.cu).  With d_dims the
// per-sequence arrays and their counts come from an earlier kernel on the stream: n_seqs and
// max_q_len are then upper bounds that size the grid, and table_offset is indexed like q_start.
// num_blocks <= 0: the pool size is unknown (llm-engine's launcher signature carries none).
template <typename T>
int prefill_launch(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                   const int* table_offset, const int* q_start, const int* q_len, const int* ctx_len, void* out,
                   int n_tokens, int n_seqs, int max_q_len, int q_heads, int kv_heads, int head_dim, int block_size,
                   int num_blocks, float scale, pkv_stream stream, const int* d_dims, bool may_allocate) {
  const char* fn = "pkv_prefill_attn";
  if (n_seqs <= 0 || n_tokens <= 0 || max_q_len <= 0) return PKV_OK;
  if (!q || !k_cache || !v_cache || !block_tables || !table_offset || !q_start || !q_len || !ctx_len || !out)
    return fail(PKV_E_ARG, "%s: null device pointer", fn);
  if (q_heads <= 0 || kv_heads <= 0)
    return fail(PKV_E_ARG, "%s: q_heads %d and kv_heads %d must be > 0", fn, q_heads, kv_heads);
  if (q_heads % kv_heads != 0)
    return fail(PKV_E_UNSUPPORTED, "%s: q_heads %d is not a multiple of kv_heads %d", fn, q_heads, kv_heads);
  if (head_dim != kHd)
    return fail(PKV_E_UNSUPPORTED, "%s: head_dim %d; the tensor-core kernel is written for head_dim %d", fn, head_dim, kHd);
  const int bsl = log2_exact(block_size);
  if (bsl < 4)
    return fail(PKV_E_UNSUPPORTED, "%s: block_size %d; needs a power of two >= 16 (one TMA box is 16 slots)", fn, block_size);
  if (!(scale > 0.f)) return fail(PKV_E_ARG, "%s: scale must be positive", fn);
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out))
    return fail(PKV_E_ARG, "%s: q, out and the K/V pools must be 16-byte aligned", fn);
  if (n_seqs > 65535) return fail(PKV_E_UNSUPPORTED, "%s: at most 65535 sequences per call", fn);
  PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
  if (!enc) return fail(PKV_E_CUDA, "%s: cuTensorMapEncodeTiled is not available from this driver", fn);

  constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
  alignas(64) CUtensorMap qmap, kmap, vmap;
  const int kv_dim = kv_heads * head_dim;
  const uint64_t pool_rows = num_blocks > 0 ? static_cast<uint64_t>(num_blocks) * block_size : (1ull << 30);
  int st = make_pool_tensor_map(&kmap, k_cache, is_bf16, kv_dim, 16, pool_rows);
  if (st != PKV_OK) return st;
  st = make_pool_tensor_map(&vmap, v_cache, is_bf16, kv_dim, 16, pool_rows);
  if (st != PKV_OK) return st;
  // q as [n_tokens][q_heads*head_dim]; rows past n_tokens read as zeros
  st = make_pool_tensor_map(&qmap, q, is_bf16, q_heads * head_dim, kQTile, static_cast<uint64_t>(n_tokens));
  if (st != PKV_OK) return st;

  auto kern = prefill_tc_kernel<T>;
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    if (e != cudaSuccess) return fail(PKV_E_CUDA, "%s: cannot reserve %d bytes of shared memory: %s", fn, kSmemTotal, cudaGetErrorString(e));
    configured_device = dev;
  }
  PrefillArgs a;
  a.block_tables = block_tables; a.table_offset = table_offset;
  a.q_start = q_start; a.q_len = q_len; a.ctx_len = ctx_len;
  a.out = out;
  a.q_heads = q_heads; a.kv_heads = kv_heads; a.group = q_heads / kv_heads;
  a.block_size = block_size; a.bs_log2 = bsl;
  a.scale = scale;
  a.n_qtiles_max = (max_q_len + kQTile - 1) / kQTile;
  a.n_seqs = n_seqs;
  const long long n_items = static_cast<long long>(n_seqs) * a.n_qtiles_max * q_heads;
  if (n_items > 0x7fffffffll) return fail(PKV_E_UNSUPPORTED, "%s: %lld work items; at most 2^31 - 1 per call", fn, n_items);
  a.n_items = static_cast<int>(n_items);
  a.dims = d_dims;
  a.host_err = error_mirror(may_allocate);
  const TicketPair tp = ticket_pair_for(static_cast<cudaStream_t>(stream), dev);
  a.ticket = tp.ticket;
  a.done = tp.done;
  // Persistent blocks: two per SM, or one per item if there are fewer.
  static thread_local int sms = 0;
  if (!sms) {
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  // PKV_PREFILL_BLOCKS_PER_SM = 1: half the persistent grid (a measurement aid: what one block per SM does alone)
  static const int per_sm = [] { const char* e = std::getenv("PKV_PREFILL_BLOCKS_PER_SM"); return (e && e[0] == '1') ? 1 : 2; }();
  const int blocks = static_cast<int>(std::min<long long>(n_items, static_cast<long long>(per_sm) * sms));
  launch_pdl(kern, dim3(blocks), dim3(kThreads), kSmemTotal, static_cast<cudaStream_t>(stream), a, qmap, kmap, vmap);
  return check_launch("prefill_tc_kernel");
}

template int prefill_launch<__nv_bfloat16>(const void*, const void*, const void*, const int*, const int*, const int*,
                                           const int*, const int*, void*, int, int, int, int, int, int, int, int, float,
                                           pkv_stream, const int*, bool);
template int prefill_launch<__half>(const void*, const void*, const void*, const int*, const int*, const int*, const int*,
                                    const int*, void*, int, int, int, int, int, int, int, int, float, pkv_stream,
                                    const int*, bool);

namespace {

template <typename T>
int prefill_impl(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                 const int* table_offset, const int* q_start, const int* q_len, const int* ctx_len, void* out,
                 int n_tokens, int n_seqs, int max_q_len, int q_heads, int kv_heads, int head_dim, int block_size,
                 int num_blocks, float scale, pkv_stream stream) {
  if (n_seqs <= 0 || n_tokens <= 0 || max_q_len <= 0) return PKV_OK;
  const int st = check_error_mirror("pkv_prefill_attn");
  if (st != PKV_OK) return st;
  if (num_blocks <= 0) return fail(PKV_E_ARG, "pkv_prefill_attn: num_blocks %d must be > 0", num_blocks);
  return prefill_launch<T>(q, k_cache, v_cache, block_tables, table_offset, q_start, q_len, ctx_len, out, n_tokens,
                           n_seqs, max_q_len, q_heads, kv_heads, head_dim, block_size, num_blocks, scale, stream,
                           nullptr, true);
}

}  // namespace

// Reads and clears this file's share of the device error word (pkv_debug_device_flags).
int prefill_read_flags(unsigned int* flags) {
  unsigned int v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_pkv_prefill_error, sizeof(v));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_pkv_prefill_error, &zero, sizeof(zero));
  if (e != cudaSuccess) return fail(PKV_E_CUDA, "pkv_debug_device_flags: %s", cudaGetErrorString(e));
  *flags = v;
  return PKV_OK;
}

}  // namespace pkv

extern "C" {
int pkv_prefill_attn_bf16(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                          const int* table_offset, const int* q_start, const int* q_len, const int* ctx_len,
                          void* out, int n_tokens, int n_seqs, int max_q_len, int q_heads, int kv_heads,
                          int head_dim, int block_size, int num_blocks, float scale, pkv_stream stream) {
  return pkv::prefill_impl<__nv_bfloat16>(q, k_cache, v_cache, block_tables, table_offset, q_start, q_len, ctx_len, out,
                                          n_tokens, n_seqs, max_q_len, q_heads, kv_heads, head_dim, block_size,
                                          num_blocks, scale, stream);
}
int pkv_prefill_attn_f16(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                         const int* table_offset, const int* q_start, const int* q_len, const int* ctx_len,
                         void* out, int n_tokens, int n_seqs, int max_q_len, int q_heads, int kv_heads,
                         int head_dim, int block_size, int num_blocks, float scale, pkv_stream stream) {
  return pkv::prefill_impl<__half>(q, k_cache, v_cache, block_tables, table_offset, q_start, q_len, ctx_len, out,
                                   n_tokens, n_seqs, max_q_len, q_heads, kv_heads, head_dim, block_size, num_blocks,
                                   scale, stream);
}
}
