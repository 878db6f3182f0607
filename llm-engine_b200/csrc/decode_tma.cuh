// Paged decode attention, TMA variant (sm_100a): 16-bit K/V, head_dim 64 or 128,
// GQA group <= 16, block_size a multiple of 16.
//
// Work unit = (token, key range) x kv head.  Every WARP is an independent worker:
// it owns a private ring of shared-memory stages, fetches its own units, and
// finishes them on its own -- there is no block-wide barrier and no cross-warp
// merge anywhere in the kernel, so the look-ups at the start of a unit and the
// store / split-K arrival at its end stall one warp out of the twelve or sixteen on
// the SM while the others keep the memory system busy.
//
//   loads   one lane issues TMA box copies (cp.async.bulk.tensor.2d: 16 slots x 128
//           bytes, 128-byte swizzle) through the block table, one box per 16 keys for
//           K and for V, completing on the stage's mbarrier.  The issue pointer runs
//           NSTAGES slabs ahead of the math and crosses unit boundaries, so the ring
//           never drains between units.  Table entries are fetched 32 boxes at a
//           time (one coalesced load) and handed out by shuffle.
//   math    keys are the M dimension of mma.sync m16n8k16 and the group's query heads
//           the N dimension (S^T = K Q^T, O^T = V^T P^T): a group of up to 8 heads
//           wastes no tensor-core rows, and the online-softmax state of a head lives
//           in the thread that owns its accumulator column -- no cross-lane traffic
//           for the rescale, three shuffles per slab for the running maximum, one
//           movmatrix per 8x8 block of P.
//   finish  a unit that covers its token's whole history writes the output rows; any
//           other writes its split-K partial, fire and forget; decode_combine_kernel
//           (decode_attn.cuh) merges the partials afterwards.
//
// Every mbarrier wait is bounded; a wait that runs out records a flag (device word and the
// host's pinned word) and the warp winds down instead of spinning.  Blocks are persistent and all
// start together, so a launch ends within a few wait limits whatever happens; a recorded flag
// does not stop later launches.
#pragma once

#include "decode_attn.cuh"
#include "tma_util.hpp"

namespace pkv {

constexpr unsigned kErrProducerWait = 1u, kErrConsumerWait = 2u;

constexpr int kBoxBytes = 16 * 128;

struct WarpGroup {
  static __device__ __forceinline__ void sync() { __syncwarp(); }
  static __device__ __forceinline__ int size() { return 32; }
  static __device__ __forceinline__ int tid() { return threadIdx.x & 31; }
};

template <int D, int MT, int NSTAGES, int WARPS> struct TmaSmem {
  static constexpr int kHalves = D / 64;
  static constexpr int kKBytes = MT * kHalves * kBoxBytes;  // K part of a stage; V follows
  static constexpr int kStageBytes = 2 * kKBytes;
  static constexpr int kWarpBytes = NSTAGES * kStageBytes;
  static constexpr int kBytes = WARPS * kWarpBytes + 1024;
};

// TOK = 1: a unit serves one token.  TOK = 4: a unit serves up to four tokens whose sequences
// share the blocks of its key range (a common prompt prefix): the K/V slab is fetched once and
// the tokens' heads sit side by side in the N dimension (NT / TOK head tiles per token); every
// token gets its own split-K partial.  Such units come from the shared-prefix planner as
// SharedItem records (decode_plan.hpp).
// FUSED_APPEND: the unit that reaches a token's newest key takes that row from the step's k / v
// inputs and writes it to the pool (DecodeArgs::new_k); a separate instantiation, so that the
// plain kernel carries none of it.
// CLUSTER: small steps.  The launch is a grid of thread-block clusters, one cluster per (token, kv
// head); the history is cut into as many equal ranges as the cluster has warps (fewer when it is
// short), warp w of block r takes range w * blocks + r, and the split-K merge happens inside the
// launch.  Block r of the cluster owns query heads r, r + blocks, ... of the group: a warp that has
// finished its range sends, for every head, that head's 64 sums and (maximum, sum) to the head's
// owner -- st.async stores into the owner's landing area in shared memory, each completing bytes
// on the owner's mbarrier -- and every block, once its barrier has counted all the bytes its heads
// expect, folds them from its own shared memory into the output rows.  No plan, no workspace, no
// merge kernel, no cluster-wide barrier after the first (which only publishes the mbarriers): the
// ranges and the byte counts follow from token_pos alone.
constexpr int kClusterRecord = 68 * 4;   // one (head, range) record in a landing area: 64 sums, maximum, sum, 8 bytes unused
// Landing area of a block: records for ceil(8 / blocks) heads x (4 warps x blocks) ranges; the
// cluster sizes the launcher offers (2, 3, 4, 8) need at most 3 x 12 of them.
constexpr int kClusterLandBytes = 36 * kClusterRecord + 96;
__host__ __device__ constexpr bool cluster_size_ok(int cs) { return cs == 2 || cs == 3 || cs == 4 || cs == 8; }

__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// 16 bytes into another block's shared memory; the bytes count on that block's mbarrier when they land.
__device__ __forceinline__ void cluster_push4(uint32_t dst_cluster_addr, float4 v, uint32_t bar_cluster_addr) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];\n" ::"r"(dst_cluster_addr),
               "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(bar_cluster_addr)
               : "memory");
}

template <typename T, int D, int NT, int MT, int NSTAGES, int WARPS, int MIN_BLOCKS, int TOK = 1, bool FUSED_APPEND = false,
          bool CLUSTER = false>
__global__ void __launch_bounds__(WARPS * 32, MIN_BLOCKS)
    decode_tma_kernel(const DecodeArgs a, const __grid_constant__ CUtensorMap kmap,
                      const __grid_constant__ CUtensorMap vmap) {
  using S = TmaSmem<D, MT, NSTAGES, WARPS>;
  static_assert(TOK == 1 || TOK == 4, "a shared unit holds four tokens");
  static_assert(NT % TOK == 0, "whole head tiles per token");
  static_assert(!CLUSTER || TOK == 1, "cluster launches take ordinary tokens");
  static_assert(!CLUSTER || (NT == 1 && D == 64), "the cluster form is written for up to 8 heads of 64 dims per kv head");
  static_assert(!CLUSTER || (8 * NT * D + 32 * NT) * 4 <= S::kWarpBytes, "a warp's partial must fit its ring");
  constexpr int NTG = NT / TOK;   // head tiles (8 heads each) per token
  constexpr int KS = D / 16;
  constexpr int HALVES = S::kHalves;
  constexpr int SLAB = 16 * MT;
  constexpr float kLog2e = 1.4426950408889634f;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long full_bar[WARPS * NSTAGES];
  __shared__ __align__(8) unsigned long long land_bar;     // cluster launches: counts the bytes this block's heads expect

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const uint32_t ring0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ring = ring0 + warp * S::kWarpBytes;
  unsigned char* ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
  const uint32_t bars = smem_u32(&full_bar[warp * NSTAGES]);
  const float sl2 = a.scale * kLog2e;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NSTAGES; ++s) mbar_init(bars + 8 * s, 1);
    mbar_fence_init();
  }
  __syncwarp();

  // Everything above touched only this block's shared memory.  What follows reads the plan and the
  // step's index arrays, which are complete before the predecessor on the stream even starts (they
  // are built once per step, ahead of every layer's launches, by copies or by kernels that do not
  // release their dependents early), so the look-ups that lead to a unit's first load -- item, sequence,
  // table offset, table entries -- run while the predecessor is still finishing.  What the predecessor
  // itself may have written (pool rows appended by the preceding launch, q and the new k / v rows, the
  // workspace the previous merge has finished with) is touched only after griddepcontrol.wait, which
  // every lane executes in issue_next() right before the warp's first load is issued -- or, with the
  // append inside this launch, only before the unit's q rows are read (see there): the pool rows it
  // loads are then all from earlier steps.
  pdl_launch_dependents();
  if (lane == 0) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&kmap) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&vmap) : "memory");
  }
  bool waited = false;
  // Cluster launches: this warp's one unit, from the token's position alone (a step constant).
  int c_token = 0, c_kvh = 0, c_begin = 0, c_len = 0, c_nsplits = 1, c_split = 0;
  uint32_t c_rank = 0, c_size = 1;
  if constexpr (CLUSTER) {
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(c_rank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(c_size));
    const int pair = blockIdx.x / c_size;                  // clusters are runs of consecutive blocks
    c_token = pair / a.kv_heads;
    c_kvh = pair - c_token * a.kv_heads;
    const int len = max(__ldg(a.token_pos + c_token), 0) + 1;
    const int nw = WARPS * static_cast<int>(c_size);
    const int range = (((len + nw - 1) / nw + SLAB - 1) / SLAB) * SLAB;   // whole slabs per warp
    c_nsplits = (len + range - 1) / range;
    c_split = warp * static_cast<int>(c_size) + static_cast<int>(c_rank);   // neighbouring ranges on different SMs
    c_begin = c_split * range;
    c_len = min(range, len - c_begin);                     // <= 0: no unit for this warp
    if (c_nsplits > 1) {                                   // the same for every thread of the cluster
      if (threadIdx.x == 0) {
        const int owned = (a.group - static_cast<int>(c_rank) + static_cast<int>(c_size) - 1) / static_cast<int>(c_size);
        mbar_init(smem_u32(&land_bar), 1);
        mbar_fence_init();
        // all of this block's heads' records, from every range; a block that owns no head (fewer heads
        // than blocks) expects nothing and its barrier completes at once
        mbar_arrive_expect_tx(smem_u32(&land_bar), static_cast<uint32_t>(owned * c_nsplits * kClusterRecord));
      }
      // publish the barriers: nobody sends before every block has armed its own (waited for below,
      // right before the first send, by which time it has long completed)
      __syncwarp();
      asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    }
  }
  const int n_items = CLUSTER ? 0 : (TOK > 1 ? a.n_shared : (a.direct ? a.n_tokens : a.header->n_items));
  const int total = CLUSTER ? (c_len > 0 ? 1 : 0) : n_items * a.kv_heads;
  const int gw = CLUSTER ? 0 : blockIdx.x * WARPS + warp, GW = CLUSTER ? 1 : gridDim.x * WARPS;

  // ---------------------------- issue side ----------------------------
  int iu = gw - GW;             // unit the issue pointer is in (advanced before first use)
  int i_nslabs = 0, i_slab = 0, i_kvbeg = 0, i_len = 0, i_x0 = 0;
  const int* i_tbl = nullptr;
  int i_ent = 0, i_ent_base = -64;   // this lane's block-table entry for box i_ent_base + lane
  uint32_t n_issued = 0, n_consumed = 0;

  // Issues the next slab of this warp's unit sequence, if there is one.
  auto issue_next = [&]() -> bool {
    while (i_slab >= i_nslabs) {
      iu += GW;
      if (iu >= total) { iu = total; return false; }
      const int item = iu / a.kv_heads, kvh = CLUSTER ? c_kvh : iu - item * a.kv_heads;
      int token, part;
      if constexpr (CLUSTER) {
        token = c_token;
        i_kvbeg = c_begin;
        i_len = c_len;
        part = 0;
      } else if constexpr (TOK > 1) {
        const int4 h0 = __ldg(a.shared_items + 3 * item), tk = __ldg(a.shared_items + 3 * item + 1);
        i_kvbeg = h0.x;
        i_len = h0.y;
        token = tk.x;          // every token of the unit has the same blocks over this range
        part = 0;
      } else {
        load_item(a, item, token, i_kvbeg, i_len, part);
      }
      i_tbl = a.block_tables + __ldg(a.table_offset + __ldg(a.token_seq + token));
      i_nslabs = (i_len + SLAB - 1) / SLAB;
      i_slab = 0;
      i_x0 = kvh * D;
      i_ent_base = -64;
      // warm the query rows of this unit for the math side (group x D 16-bit values)
      if constexpr (TOK == 1) {
        const char* qrow = reinterpret_cast<const char*>(static_cast<const T*>(a.q) +
                                                         (static_cast<size_t>(token) * a.q_heads + kvh * a.group) * D);
        if (lane * 128 < a.group * D * 2) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(qrow + lane * 128));
      }
    }
    const int box0 = i_slab * MT;
    if (box0 + MT > i_ent_base + 32) {   // fetch the entries of the next 32 boxes in one coalesced load
      i_ent_base = box0;
      const int rel = (box0 + lane) * 16;
      i_ent = rel < i_len ? __ldg(i_tbl + ((i_kvbeg + rel) >> a.bs_log2)) : 0;
    }
    int ent[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) ent[m] = __shfl_sync(0xffffffffu, i_ent, box0 + m - i_ent_base);
    if constexpr (!FUSED_APPEND) {
      if (!waited) {
        pdl_wait();
        waited = true;
      }
    }
    // The slot's previous contents were read with ordinary loads (ldmatrix) by all
    // lanes; order those before the asynchronous-proxy write that refills it.
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      const uint32_t slot = n_issued % NSTAGES;
      const uint32_t fb = bars + 8 * slot;
      const uint32_t st = ring + slot * S::kStageBytes;
      const int rel0 = i_slab * SLAB;
      int nvalid = 0;
#pragma unroll
      for (int m = 0; m < MT; ++m) nvalid += (rel0 + 16 * m < i_len) ? 1 : 0;
      mbar_arrive_expect_tx(fb, static_cast<uint32_t>(nvalid) * 2u * HALVES * kBoxBytes);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (rel0 + 16 * m < i_len) {
          const int key0 = i_kvbeg + rel0 + 16 * m;
          const int y = (ent[m] << a.bs_log2) + (key0 & (a.block_size - 1));
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            const uint32_t dst = st + (m * HALVES + h) * kBoxBytes;
            tma_load_2d(dst, &kmap, i_x0 + 64 * h, y, fb);
            tma_load_2d(dst + S::kKBytes, &vmap, i_x0 + 64 * h, y, fb);
          }
        }
      }
    }
    ++n_issued;
    ++i_slab;
    return true;
  };

  // ---------------------------- math side -----------------------------
  const int mi = lane >> 3, r8 = lane & 7;
  bool more = true;
  for (int cu = gw; cu < total; cu += GW) {
    const int item = cu / a.kv_heads, kvh = CLUSTER ? c_kvh : cu - item * a.kv_heads;
    int token, kv_begin, kv_len, part;
    int toks[TOK], parts[TOK], n_tok = 1;
    if constexpr (CLUSTER) {
      token = c_token; kv_begin = c_begin; kv_len = c_len;
      part = c_nsplits > 1 ? c_split : -1;
      toks[0] = token; parts[0] = part;
    } else if constexpr (TOK > 1) {
      const int4 h0 = __ldg(a.shared_items + 3 * item), tk = __ldg(a.shared_items + 3 * item + 1),
                 pt = __ldg(a.shared_items + 3 * item + 2);
      kv_begin = h0.x; kv_len = h0.y; n_tok = h0.z;
      toks[0] = tk.x; toks[1] = tk.y; toks[2] = tk.z; toks[3] = tk.w;
      parts[0] = pt.x; parts[1] = pt.y; parts[2] = pt.z; parts[3] = pt.w;
      token = toks[0]; part = parts[0];
    } else {
      load_item(a, item, token, kv_begin, kv_len, part);
      toks[0] = token; parts[0] = part;
    }
    const int n_slabs = (kv_len + SLAB - 1) / SLAB;

    while (more && n_issued - n_consumed < NSTAGES) more = issue_next();

    if constexpr (FUSED_APPEND) {
      // With the append inside this launch the loads issued above fetch only rows of EARLIER steps (the
      // newest row comes from the step's k / v below): they need not wait for the predecessor, which
      // cannot be writing them -- a step's launches are preceded by that step's uploads or planning,
      // which complete before anything behind them starts.  What the predecessor does produce -- q, the
      // new k / v rows -- and everything this launch writes comes after this wait.
      if (!waited) {
        pdl_wait();
        waited = true;
      }
    }
    // Q^T fragments (B operand): rows = dims, columns = heads of the group.
    uint32_t qb[KS][NT][2];
    {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int ti = nt / NTG;                    // which token of the unit this head tile belongs to
        const T* qbase = static_cast<const T*>(a.q) + (static_cast<size_t>(toks[ti]) * a.q_heads + kvh * a.group) * D;
        const int head = 8 * (nt % NTG) + g;
        const bool hv = head < a.group && ti < n_tok;
        const uint32_t* qrow = reinterpret_cast<const uint32_t*>(qbase + static_cast<size_t>(head) * D);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          qb[ks][nt][0] = hv ? __ldg(qrow + ks * 8 + c) : 0u;
          qb[ks][nt][1] = hv ? __ldg(qrow + ks * 8 + 4 + c) : 0u;
        }
      }
    }
    float o[KS][NT][4];
    float m_run[NT][2], l_run[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      m_run[nt][0] = m_run[nt][1] = -INFINITY;
      l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
      for (int dm = 0; dm < KS; ++dm) o[dm][nt][0] = o[dm][nt][1] = o[dm][nt][2] = o[dm][nt][3] = 0.f;
    }

    bool ok = true;
    for (int j = 0; j < n_slabs; ++j) {
      while (more && n_issued - n_consumed < NSTAGES) more = issue_next();
      const uint32_t slot = n_consumed % NSTAGES;
      if (!mbar_wait(bars + 8 * slot, (n_consumed / NSTAGES) & 1u)) {
        if (lane == 0) report_give_up(a, kErrConsumerWait);
        ok = false;
        break;
      }
      const uint32_t kst = ring + slot * S::kStageBytes;
      const uint32_t vst = kst + S::kKBytes;
      const int rows_valid = min(SLAB, kv_len - j * SLAB);
      if constexpr (TOK == 1 && FUSED_APPEND) {
        if (j == n_slabs - 1 && kv_begin + kv_len == __ldg(a.token_pos + token) + 1) {
          // Fused append: this unit ends at the token's newest key, whose row is not in the pool yet.
          // Lanes 0 .. 8 HALVES - 1 bring the 16-byte pieces of its K row, the next 8 HALVES those of
          // its V row: each goes into the slab just fetched (same swizzle as the TMA boxes) and to
          // the token's slot in the pool.
          const int rl = kv_len - 1 - j * SLAB, box = rl >> 4, r = rl & 15;
          const bool is_v = lane >= 8 * HALVES;
          const int cidx = lane - (is_v ? 8 * HALVES : 0);
          if (lane < 16 * HALVES) {
            const size_t row_off = (static_cast<size_t>(kvh) * D) * sizeof(T) + static_cast<size_t>(cidx) * 16;
            const size_t kv_row_bytes = static_cast<size_t>(a.kv_heads) * D * sizeof(T);
            const char* src = static_cast<const char*>(is_v ? a.new_v : a.new_k) + static_cast<size_t>(token) * kv_row_bytes + row_off;
            const uint4 val = __ldg(reinterpret_cast<const uint4*>(src));
            char* pool = static_cast<char*>(const_cast<void*>(is_v ? a.v_cache : a.k_cache));
            *reinterpret_cast<uint4*>(pool + static_cast<size_t>(__ldg(a.slots + token)) * kv_row_bytes + row_off) = val;
            unsigned char* dst = ring_ptr + slot * S::kStageBytes + (is_v ? S::kKBytes : 0) +
                                 (box * HALVES + (cidx >> 3)) * kBoxBytes + r * 128 + (((cidx & 7) ^ (r & 7)) << 4);
            *reinterpret_cast<uint4*>(dst) = val;
          }
          __syncwarp();
        }
      }
      if (rows_valid < SLAB) {
        // Slots past the end of the history hold whatever was there before (or were
        // never fetched): their scores are masked below, and their V rows are
        // cleared here so that 0 * garbage cannot produce a NaN.
        unsigned char* vptr = ring_ptr + slot * S::kStageBytes + S::kKBytes;
        const int nrows = SLAB - rows_valid;
        for (int i = lane; i < nrows * 8 * HALVES; i += 32) {
          const int row = rows_valid + i / (8 * HALVES);
          const int rem = i % (8 * HALVES);
          const int h = rem >> 3, ch = rem & 7;
          *reinterpret_cast<uint4*>(vptr + ((row >> 4) * HALVES + h) * kBoxBytes + (row & 15) * 128 + ch * 16) =
              make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
      }

      // S^T = K Q^T : MT m-tiles of 16 keys.
      float s[MT][NT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) s[mt][nt][0] = s[mt][nt][1] = s[mt][nt][2] = s[mt][nt][3] = 0.f;
        const int row16 = ((mi & 1) << 3) + r8;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int chunk = 2 * ks + (mi >> 1);
          const uint32_t addr = kst + (mt * HALVES + (chunk >> 3)) * kBoxBytes + row16 * 128 + (((chunk & 7) ^ r8) << 4);
          uint32_t ka[4];
          ldmatrix_x4(addr, ka[0], ka[1], ka[2], ka[3]);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma16816<T>(s[mt][nt], ka, qb[ks][nt][0], qb[ks][nt][1]);
        }
      }
      if (rows_valid < SLAB) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (16 * mt + g + 8 * (e >> 1) >= rows_valid) s[mt][nt][e] = -INFINITY;
      }
      // Online softmax, per head (thread holds heads 8nt+2c and 8nt+2c+1).
      uint32_t pb[MT][NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float mx0 = fmaxf(s[0][nt][0], s[0][nt][2]);
        float mx1 = fmaxf(s[0][nt][1], s[0][nt][3]);
#pragma unroll
        for (int mt = 1; mt < MT; ++mt) {
          mx0 = fmaxf(mx0, fmaxf(s[mt][nt][0], s[mt][nt][2]));
          mx1 = fmaxf(mx1, fmaxf(s[mt][nt][1], s[mt][nt][3]));
        }
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);
        const float al0 = exp2f((m_run[nt][0] - mn0) * sl2), al1 = exp2f((m_run[nt][1] - mn1) * sl2);
        m_run[nt][0] = mn0;
        m_run[nt][1] = mn1;
        const float ng0 = -mn0 * sl2, ng1 = -mn1 * sl2;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const float p0 = exp2f(fmaf(s[mt][nt][0], sl2, ng0)), p1 = exp2f(fmaf(s[mt][nt][1], sl2, ng1));
          const float p2 = exp2f(fmaf(s[mt][nt][2], sl2, ng0)), p3 = exp2f(fmaf(s[mt][nt][3], sl2, ng1));
          ps0 += p0 + p2;
          ps1 += p1 + p3;
          // (key g | g+8 ; heads 2c, 2c+1)  ->  (head g ; keys 2c, 2c+1): the B operand of O^T += V^T P^T
          movmatrix_trans(pb[mt][nt][0], pack2<T>(p0, p1));
          movmatrix_trans(pb[mt][nt][1], pack2<T>(p2, p3));
        }
        l_run[nt][0] = l_run[nt][0] * al0 + ps0;
        l_run[nt][1] = l_run[nt][1] * al1 + ps1;
#pragma unroll
        for (int dm = 0; dm < KS; ++dm) {
          o[dm][nt][0] *= al0;
          o[dm][nt][1] *= al1;
          o[dm][nt][2] *= al0;
          o[dm][nt][3] *= al1;
        }
      }
      // O^T += V^T P^T : m-tiles of 16 dims, k = the slab's keys.
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int row16 = ((mi >> 1) << 3) + r8;
#pragma unroll
        for (int dm = 0; dm < KS; ++dm) {
          const int chunk = 2 * dm + (mi & 1);
          const uint32_t addr = vst + (mt * HALVES + (chunk >> 3)) * kBoxBytes + row16 * 128 + (((chunk & 7) ^ r8) << 4);
          uint32_t va[4];
          ldmatrix_x4_trans(addr, va[0], va[1], va[2], va[3]);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma16816<T>(o[dm][nt], va, pb[mt][nt][0], pb[mt][nt][1]);
        }
      }
      ++n_consumed;
    }
    if constexpr (!CLUSTER) {
      if (!ok) return;  // this warp has copies in flight only into its own ring; nothing else depends on it
    }                   // (in a cluster the warp stays for the barriers; its give-up is on record)

    while (more && n_issued - n_consumed < NSTAGES) more = issue_next();  // keep loads flowing through the finish

    // ------------------------------ finish the unit ------------------------------
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        l_run[nt][0] += __shfl_xor_sync(0xffffffffu, l_run[nt][0], off);
        l_run[nt][1] += __shfl_xor_sync(0xffffffffu, l_run[nt][1], off);
      }
    }
    const int head_base = kvh * a.group;
    if (TOK == 1 && part < 0) {
      T* out = out_row<T>(a, a.out, token) + static_cast<size_t>(head_base) * D;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int h0 = 8 * nt + 2 * c;
        const float i0 = 1.f / l_run[nt][0], i1 = 1.f / l_run[nt][1];
#pragma unroll
        for (int dm = 0; dm < KS; ++dm) {
          const int d = 16 * dm + g;
          if (h0 < a.group) {
            out[static_cast<size_t>(h0) * D + d] = Elem<T>::from_f32(o[dm][nt][0] * i0);
            out[static_cast<size_t>(h0) * D + d + 8] = Elem<T>::from_f32(o[dm][nt][2] * i0);
          }
          if (h0 + 1 < a.group) {
            out[static_cast<size_t>(h0 + 1) * D + d] = Elem<T>::from_f32(o[dm][nt][1] * i1);
            out[static_cast<size_t>(h0 + 1) * D + d + 8] = Elem<T>::from_f32(o[dm][nt][3] * i1);
          }
        }
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int ti = nt / NTG;
        if (ti >= n_tok) continue;
        // the partial: to the workspace, or (cluster launches) to the start of this warp's own ring,
        // which holds no copy in flight any more -- [8 NT heads][D] sums, then (maximum, sum) per head
        float* pacc = CLUSTER ? reinterpret_cast<float*>(ring_ptr)
                              : a.part_acc + (static_cast<size_t>(parts[ti]) * a.q_heads + head_base) * D;
        float* pml = CLUSTER ? reinterpret_cast<float*>(ring_ptr) + 8 * NT * D
                             : a.part_ml + (static_cast<size_t>(parts[ti]) * a.q_heads + head_base) * 2;
        const int h0 = 8 * (nt % NTG) + 2 * c;
#pragma unroll
        for (int dm = 0; dm < KS; ++dm) {
          const int d = 16 * dm + g;
          if (h0 < a.group) {
            pacc[static_cast<size_t>(h0) * D + d] = o[dm][nt][0];
            pacc[static_cast<size_t>(h0) * D + d + 8] = o[dm][nt][2];
          }
          if (h0 + 1 < a.group) {
            pacc[static_cast<size_t>(h0 + 1) * D + d] = o[dm][nt][1];
            pacc[static_cast<size_t>(h0 + 1) * D + d + 8] = o[dm][nt][3];
          }
        }
        if (g == 0) {
          if (h0 < a.group) { pml[2 * h0] = m_run[nt][0] * sl2; pml[2 * h0 + 1] = l_run[nt][0]; }
          if (h0 + 1 < a.group) { pml[2 * h0 + 2] = m_run[nt][1] * sl2; pml[2 * h0 + 3] = l_run[nt][1]; }
        }
      }
    }
  }
  if constexpr (CLUSTER) {
    if (c_nsplits > 1) {               // the same for every thread of the cluster
      if (!waited) pdl_wait();         // warps without a range write output rows too
      asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");   // every block's landing barrier is armed
      const uint32_t land0 = ring0 + WARPS * S::kWarpBytes;                   // landing area: behind the rings
      const int ranges_max = WARPS * static_cast<int>(c_size);
      if (c_len > 0) {
        // send this warp's partial, head by head, to the heads' owners: 16 quads of sums and one with
        // (maximum, sum) per head, read back from where the unit's finish left them
        __syncwarp();
        const float* pacc = reinterpret_cast<const float*>(ring_ptr);
        const float* pml = pacc + 8 * NT * D;
        for (int i = lane; i < a.group * 17; i += 32) {
          const int h = i / 17, k = i - h * 17;
          const uint32_t owner = static_cast<uint32_t>(h) % c_size, j = static_cast<uint32_t>(h) / c_size;
          float4 v;
          if (k < 16) {
            v = *reinterpret_cast<const float4*>(pacc + h * D + 4 * k);
          } else {
            const float2 ml = *reinterpret_cast<const float2*>(pml + 2 * h);
            v = make_float4(ml.x, ml.y, 0.f, 0.f);
          }
          const uint32_t dst = land0 + (j * ranges_max + c_split) * kClusterRecord + 16 * k;
          cluster_push4(cluster_map(dst, owner), v, cluster_map(smem_u32(&land_bar), owner));
        }
      }
      // this block's heads: wait for all their records, fold them, write the rows
      if (!mbar_wait(smem_u32(&land_bar), 0u)) {
        if (threadIdx.x == 0) report_give_up(a, kErrConsumerWait);
      }
      const int owned = (a.group - static_cast<int>(c_rank) + static_cast<int>(c_size) - 1) / static_cast<int>(c_size);
      const unsigned char* land_ptr = smem_raw + (land0 - smem_u32(smem_raw));
      for (int e = threadIdx.x; e < owned * (D / 2); e += WARPS * 32) {     // one pair of dims per thread
        const int j = e / (D / 2), d = 2 * (e - j * (D / 2));
        const int h = j * static_cast<int>(c_size) + static_cast<int>(c_rank);
        const unsigned char* rec0 = land_ptr + static_cast<size_t>(j) * ranges_max * kClusterRecord;
        float m_run = -INFINITY;
#pragma unroll 4
        for (int sp = 0; sp < c_nsplits; ++sp) m_run = fmaxf(m_run, *reinterpret_cast<const float*>(rec0 + sp * kClusterRecord + 256));
        float l_run = 0.f, acc0 = 0.f, acc1 = 0.f;
#pragma unroll 4
        for (int sp = 0; sp < c_nsplits; ++sp) {
          const unsigned char* rec = rec0 + sp * kClusterRecord;
          const float2 ml = *reinterpret_cast<const float2*>(rec + 256);
          const float f = (ml.x == -INFINITY) ? 0.f : exp2f(ml.x - m_run);
          const float2 v = *reinterpret_cast<const float2*>(rec + 4 * d);
          l_run += f * ml.y;
          acc0 += f * v.x;
          acc1 += f * v.y;
        }
        const float inv = 1.f / l_run;
        T* o = out_row<T>(a, a.out, c_token) + static_cast<size_t>(c_kvh * a.group + h) * D + d;
        *reinterpret_cast<uint32_t*>(o) = pack2<T>(acc0 * inv, acc1 * inv);
      }
    }
  }
}

}  // namespace pkv
