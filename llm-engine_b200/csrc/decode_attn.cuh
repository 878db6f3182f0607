// Paged decode attention kernels (sm_100a).
//
// What they compute is ref::paged_attention_head of llm-engine
// (include/engine/ops.h:87-111) for every packed token and query head: scores of
// the query against keys 0..token_pos inclusive gathered through the sequence's
// block table, softmax, weighted sum of the values.  How they compute it:
//
//   * one thread block per work item (token, key range) x kv head; ALL query
//     heads of the GQA group share each K/V row read (the reference's baseline
//     kernel reads it once per query head, src/kernels/attention_decode.cu:45-131);
//   * 16-bit K/V: each warp streams 16-key tiles of its own through a private
//     cp.async ring in shared memory (16-byte coalesced copies, XOR-swizzled rows,
//     no block-wide barrier in the loop), feeds them to mma.sync m16n8k16 with the
//     group's query heads as the M dimension, and keeps an online softmax in
//     registers (quad shuffles for the row maximum);
//   * fp32 K/V, or any geometry the tensor-core path does not cover: a SIMT kernel
//     with the same work decomposition and fp32 arithmetic throughout;
//   * split-K: partial (max, denominator, accumulator) per item in the caller's
//     workspace, merged by a small second kernel on the same stream; nothing ever
//     waits on a flag.
#pragma once

#include "common.cuh"
#include "decode_plan.hpp"
#include "launch_util.hpp"

namespace pkv {

// Word in which kernels record a bounded wait that ran out (read and cleared by pkv_debug_device_flags).
__device__ unsigned int g_pkv_device_error = 0;

constexpr int kMaxPeers = 8;
constexpr unsigned kErrPeerWait = 8u;   // bit of the device error word: a peer's flag did not arrive in time

struct DecodeArgs {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int* block_tables;
  const int* table_offset;
  const int* token_seq;
  const int* token_pos;
  void* out;
  int n_tokens, q_heads, kv_heads, head_dim, group;
  int block_size, bs_log2;  // bs_log2 < 0 when block_size is not a power of two
  float scale;
  // plan (all null / 0 in direct mode)
  const PlanHeader* header;
  const WorkItem* items;
  const TokSplit* tok_split;
  int* counters;
  float* part_ml;
  float* part_acc;
  int direct;  // 1: item i is token i over its whole history, no workspace
  // shared-prefix units (decode_tma_kernel with TOK = 4 only): three int4 per unit
  const int4* shared_items;
  int n_shared;
  // Where a token's output row lives: out + token * out_row_elems + out_col0 + head * head_dim.
  // (q_heads * head_dim and 0 unless the heads of a row are spread over several GPUs.)
  long long out_row_elems;
  int out_col0;
  // Head-sharded exchange, done by the merge kernel (n_peers = 0: off).  peer_out[p] is rank p's
  // full output buffer (this rank's own is peer_out[my_rank] == out), peer_flags[p] an array of
  // n_peers ints on rank p; this rank writes `epoch` to peer_flags[p][my_rank] once all its rows
  // have been stored everywhere, and waits until its own flags all show `epoch`.
  void* peer_out[kMaxPeers];
  int* peer_flags[kMaxPeers];
  int n_peers, my_rank, epoch;
  // Append fused into the attention (decode_tma_kernel only; null = off): the unit that reaches a
  // token's newest key takes that key's K/V row from new_k / new_v [n_tokens][kv_heads*head_dim]
  // instead of the pool and writes it to pool row slots[token].  k_cache / v_cache are written.
  const void* new_k;
  const void* new_v;
  const int* slots;
  unsigned int* host_err;   // pinned host word that also receives a give-up (null: none)
  unsigned long long pool_rows;   // slots the K/V tensor maps cover (the pool size when the caller gave it, else a bound)
};

// Records a bounded wait that ran out: in the device word, and in the host's pinned word if the
// launch was given one, so that the caller's next call can report it without synchronising.
__device__ __forceinline__ void report_give_up(const DecodeArgs& a, unsigned int bit) {
  atomicOr(&g_pkv_device_error, bit);
  if (a.host_err) {
    *reinterpret_cast<volatile unsigned int*>(a.host_err) = bit;
    __threadfence_system();
  }
}

// Output row of (token, head 0) under the layout above.
template <typename T>
__device__ __forceinline__ T* out_row(const DecodeArgs& a, void* base, int token) {
  return static_cast<T*>(base) + static_cast<size_t>(token) * a.out_row_elems + a.out_col0;
}

constexpr int kDecodeThreads = 128;
constexpr int kDecodeWarps = 4;
constexpr int kTileKeys = 16;

__device__ __forceinline__ int64_t slot_of(const int* tbl, int pos, int block_size, int bs_log2) {
  if (bs_log2 >= 0) return (static_cast<int64_t>(__ldg(tbl + (pos >> bs_log2))) << bs_log2) + (pos & (block_size - 1));
  return static_cast<int64_t>(__ldg(tbl + pos / block_size)) * block_size + pos % block_size;
}

// exp in the domain the kernel's running maximum lives in: base 2 for the
// tensor-core path (scores are pre-multiplied by log2 e), natural for fp32.
template <bool LOG2> __device__ __forceinline__ float softmax_exp(float x) {
  if (LOG2) return exp2f(x);
  return expf(x);
}

// Merges the per-warp partial results of `rows` query heads (first one is
// head0 of the token) held in shared memory and stores either the final output
// rows or this item's split-K partial.
//   sm_m, sm_l : [kDecodeWarps][RS]      running max / denominator per warp and row
//   sm_o       : [kDecodeWarps][RS][ldo] unnormalised accumulators   (RS = rows per warp, 8 or 16)
// Must be called by every thread of the group `G` (the whole block, or the math
// warps of a warp-specialised block) after a G::sync(); ends with one.
struct BlockGroup {
  static __device__ __forceinline__ void sync() { __syncthreads(); }
  static __device__ __forceinline__ int size() { return blockDim.x; }
  static __device__ __forceinline__ int tid() { return threadIdx.x; }
};
// The first kDecodeWarps warps of a block whose remaining warps do other work:
// they meet on named barrier 1 and leave barrier 0 (__syncthreads) alone.
struct MathWarpsGroup {
  static __device__ __forceinline__ void sync() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }
  static __device__ __forceinline__ int size() { return 128; }
  static __device__ __forceinline__ int tid() { return threadIdx.x; }
};

template <typename T, bool LOG2, typename G = BlockGroup, int RS = 16>
__device__ __forceinline__ void merge_warps_and_store(const DecodeArgs& a, int token, int head0, int rows, int part,
                                                      const float* sm_m, const float* sm_l, const float* sm_o,
                                                      int ldo, float* sm_w /*[kDecodeWarps+2][16]*/) {
  const int D = a.head_dim;
  const int tid = threadIdx.x;
  if (tid < rows) {
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) m = fmaxf(m, sm_m[w * RS + tid]);
    float l = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float mw = sm_m[w * RS + tid];
      const float f = (mw == -INFINITY) ? 0.f : softmax_exp<LOG2>(mw - m);
      sm_w[w * 16 + tid] = f;
      l += f * sm_l[w * RS + tid];
    }
    sm_w[kDecodeWarps * 16 + tid] = m;
    sm_w[(kDecodeWarps + 1) * 16 + tid] = l;
  }
  G::sync();
  for (int idx = tid; idx < rows * D; idx += G::size()) {
    const int r = idx / D, d = idx - r * D;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) acc += sm_w[w * 16 + r] * sm_o[(w * RS + r) * ldo + d];
    const int head = head0 + r;
    if (part < 0) {
      const float l = sm_w[(kDecodeWarps + 1) * 16 + r];
      out_row<T>(a, a.out, token)[static_cast<size_t>(head) * D + d] = Elem<T>::from_f32(acc / l);
    } else {
      a.part_acc[(static_cast<size_t>(part) * a.q_heads + head) * D + d] = acc;
    }
  }
  if (part >= 0 && tid < rows) {
    float* ml = a.part_ml + (static_cast<size_t>(part) * a.q_heads + head0 + tid) * 2;
    ml[0] = sm_w[kDecodeWarps * 16 + tid];
    ml[1] = sm_w[(kDecodeWarps + 1) * 16 + tid];
  }
  G::sync();
}

// Split-K merge.  A token whose history was cut into several work items has one
// partial (running max, denominator, unnormalised accumulator) per item in the
// workspace; this kernel, launched right after the attention kernel on the same
// stream, folds them into the output rows.  Keeping the merge out of the attention
// kernel keeps fences, atomics and dependent L2 round trips off its critical path.
//
// One thread block per (token, kv head) that was split, one thread per
// (head, 4 dims).  The partials sit in L2 and a round trip costs several hundred
// cycles, so a thread issues the loads of up to sixteen splits (max/denominator pair
// and a 16-byte slice of the accumulator) before it touches any of them, and folds
// batches together with the usual rescale.
constexpr int kCombineThreads = 128;
constexpr int kCombineBatch = 16;

// Folds the partials of (token, head) for dims 4 d4 .. 4 d4 + 3 and returns the normalised values.
template <bool LOG2>
__device__ __forceinline__ float4 merge_partials4(const DecodeArgs& a, const TokSplit ts, int head, int d4, int D) {
  constexpr int B = kCombineBatch;
  float m_run = -INFINITY, l_run = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < ts.nsplits; s0 += B) {
    float2 ml[B];
    float4 v[B];
#pragma unroll
    for (int i = 0; i < B; ++i) {
      if (s0 + i < ts.nsplits) {
        const size_t p = static_cast<size_t>(ts.part_base + s0 + i) * a.q_heads + head;
        ml[i] = __ldcg(reinterpret_cast<const float2*>(a.part_ml + p * 2));
        v[i] = __ldcg(reinterpret_cast<const float4*>(a.part_acc + p * D) + d4);
      } else {
        ml[i] = make_float2(-INFINITY, 0.f);
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    float mb = m_run;
#pragma unroll
    for (int i = 0; i < B; ++i) mb = fmaxf(mb, ml[i].x);
    const float f0 = (m_run == -INFINITY) ? 0.f : softmax_exp<LOG2>(m_run - mb);
    l_run *= f0;
    acc.x *= f0; acc.y *= f0; acc.z *= f0; acc.w *= f0;
#pragma unroll
    for (int i = 0; i < B; ++i) {
      const float f = (ml[i].x == -INFINITY) ? 0.f : softmax_exp<LOG2>(ml[i].x - mb);
      l_run += f * ml[i].y;
      acc.x += f * v[i].x; acc.y += f * v[i].y; acc.z += f * v[i].z; acc.w += f * v[i].w;
    }
    m_run = mb;
  }
  const float inv = 1.f / l_run;
  return make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
}

template <typename T, bool LOG2>
__global__ void __launch_bounds__(kCombineThreads) decode_combine_kernel(const DecodeArgs a) {
  pdl_launch_dependents();
  const int D = a.head_dim;
  const int pairs = a.n_tokens * a.kv_heads;
  // The split record of this block's first (token, kv head) is part of the plan, which was complete
  // before the attention kernel started: fetch it while that kernel is still finishing.
  TokSplit ts_first{0, 0};
  if (static_cast<int>(blockIdx.x) < pairs) ts_first = a.tok_split[blockIdx.x / a.kv_heads];
  pdl_wait();  // the attention kernel's partials
  for (int pr = blockIdx.x; pr < pairs; pr += gridDim.x) {
    const int token = pr / a.kv_heads, kvh = pr - token * a.kv_heads;
    const TokSplit ts = pr == static_cast<int>(blockIdx.x) ? ts_first : a.tok_split[token];
    if (ts.nsplits <= 1 && a.n_peers == 0) continue;
    const int head0 = kvh * a.group;
    if (a.n_peers > 0) {
      // Head-sharded exchange (16-bit outputs, head_dim a multiple of 4): every row of this rank's
      // heads goes to every rank's full output buffer, 8 bytes at a time over NVLink.
      if constexpr (sizeof(T) == 2) {
        const int D4 = D >> 2;
        for (int idx = threadIdx.x; idx < a.group * D4; idx += kCombineThreads) {
          const int r = idx / D4, d4 = idx - r * D4;
          const int head = head0 + r;
          const size_t off = static_cast<size_t>(head) * D + 4 * d4;
          uint2 packed;
          if (ts.nsplits <= 1) {
            packed = *reinterpret_cast<const uint2*>(out_row<T>(a, a.out, token) + off);   // the attention kernel wrote it here
          } else {
            const float4 r4 = merge_partials4<LOG2>(a, ts, head, d4, D);
            packed.x = pack2<T>(r4.x, r4.y);
            packed.y = pack2<T>(r4.z, r4.w);
          }
          for (int p = 0; p < a.n_peers; ++p) {
            if (p == a.my_rank && ts.nsplits <= 1) continue;
            *reinterpret_cast<uint2*>(out_row<T>(a, a.peer_out[p], token) + off) = packed;
          }
        }
      }
    } else if ((D & 3) == 0) {
      const int D4 = D >> 2;
      for (int idx = threadIdx.x; idx < a.group * D4; idx += kCombineThreads) {
        const int r = idx / D4, d4 = idx - r * D4;
        const int head = head0 + r;
        const float4 r4 = merge_partials4<LOG2>(a, ts, head, d4, D);
        T* o = out_row<T>(a, a.out, token) + static_cast<size_t>(head) * D + 4 * d4;
        if (sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(o) & 7) == 0) {   // one 8-byte store instead of four 2-byte ones
          uint2 packed = make_uint2(0u, 0u);
          if constexpr (sizeof(T) == 2) {
            packed.x = pack2<T>(r4.x, r4.y);
            packed.y = pack2<T>(r4.z, r4.w);
          }
          *reinterpret_cast<uint2*>(o) = packed;
        } else {
          o[0] = Elem<T>::from_f32(r4.x);
          o[1] = Elem<T>::from_f32(r4.y);
          o[2] = Elem<T>::from_f32(r4.z);
          o[3] = Elem<T>::from_f32(r4.w);
        }
      }
    } else {
      for (int idx = threadIdx.x; idx < a.group * D; idx += kCombineThreads) {
        const int r = idx / D, d = idx - r * D;
        const int head = head0 + r;
        float m = -INFINITY;
        for (int s = 0; s < ts.nsplits; ++s)
          m = fmaxf(m, __ldcg(a.part_ml + (static_cast<size_t>(ts.part_base + s) * a.q_heads + head) * 2));
        float acc = 0.f, l = 0.f;
        for (int s = 0; s < ts.nsplits; ++s) {
          const size_t p = static_cast<size_t>(ts.part_base + s) * a.q_heads + head;
          const float f = softmax_exp<LOG2>(__ldcg(a.part_ml + p * 2) - m);
          l += f * __ldcg(a.part_ml + p * 2 + 1);
          acc += f * __ldcg(a.part_acc + p * D + d);
        }
        out_row<T>(a, a.out, token)[static_cast<size_t>(head) * D + d] = Elem<T>::from_f32(acc / l);
      }
    }
  }
  if (a.n_peers > 0) {
    // Tell every rank that this rank's rows are in its buffer, and leave only when every rank has
    // told this one: the kernel's completion then means the full output is here.  Stores to the
    // peers are made visible system-wide before the block counts itself done; the last block to do
    // so raises the flags and waits, with a bound, for the others'.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int done = atomicAdd(a.counters, 1);
      if (done == static_cast<int>(gridDim.x) - 1) {
        a.counters[0] = 0;                                   // ready for the next launch
        int* mine = a.peer_flags[a.my_rank];
        // epoch 0: count the calls on the device (slot n_peers of this rank's own flags), so that a
        // captured CUDA graph can be replayed; every rank makes the same calls and counts alike.
        const int epoch = a.epoch != 0 ? a.epoch : (mine[a.n_peers] += 1);
        __threadfence_system();
        for (int p = 0; p < a.n_peers; ++p)
          asm volatile("st.release.sys.global.s32 [%0], %1;\n" ::"l"(a.peer_flags[p] + a.my_rank), "r"(epoch) : "memory");
        for (int p = 0; p < a.n_peers; ++p) {
          int seen = 0;
          unsigned spins = 0;
          for (;;) {
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];\n" : "=r"(seen) : "l"(mine + p) : "memory");
            if (seen - epoch >= 0) break;
            if (++spins > (1u << 23)) {                      // about two seconds: the peer is not coming
              report_give_up(a, kErrPeerWait);
              break;
            }
            __nanosleep(200);
          }
        }
      }
    }
  }
}

__device__ __forceinline__ void load_item(const DecodeArgs& a, int item, int& token, int& kv_begin, int& kv_len, int& part) {
  if (a.direct) {
    token = item;
    kv_begin = 0;
    kv_len = __ldg(a.token_pos + item) + 1;
    part = -1;
  } else {
    const int4 it = __ldg(reinterpret_cast<const int4*>(a.items) + item);
    token = it.x;
    kv_begin = it.y;
    kv_len = it.z;
    part = it.w;
  }
}

// ============================================================================
// Tensor-core path: 16-bit K/V, head_dim D in {64, 128}, group <= 16,
// block_size a power of two.
// ============================================================================
template <int D, int STAGES> struct MmaSmem {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTileBytes = kTileKeys * kRowBytes;            // one of K or V
  static constexpr int kStageBytes = 2 * kTileBytes;                  // K then V
  static constexpr int kWarpBytes = STAGES * kStageBytes;
  static constexpr int kPipeBytes = kDecodeWarps * kWarpBytes;
  static constexpr int kLdo = D + 4;
  static constexpr int kMergeBytes = (kDecodeWarps * 16 * kLdo + 2 * kDecodeWarps * 16 + (kDecodeWarps + 2) * 16) * 4;
  static constexpr int kBytes = (kPipeBytes > kMergeBytes ? kPipeBytes : kMergeBytes) + 16;
};

template <typename T, int D, int STAGES, int MIN_BLOCKS>
__global__ void __launch_bounds__(kDecodeThreads, MIN_BLOCKS) decode_mma_kernel(const DecodeArgs a) {
  using S = MmaSmem<D, STAGES>;
  constexpr int KS = D / 16;             // k-steps of Q.K^T, and pairs of dim-tiles of P.V
  constexpr int CH = D / 8;              // 16-byte chunks per K/V row
  constexpr int ROWS_PER_PASS = 32 / CH; // rows one warp-wide cp.async covers
  constexpr int PASSES = kTileKeys / ROWS_PER_PASS;
  constexpr float kLog2e = 1.4426950408889634f;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const uint32_t warp_smem = smem_u32(smem_raw) + warp * S::kWarpBytes;
  const int kv_dim = a.kv_heads * D;
  const float sl2 = a.scale * kLog2e;

  pdl_launch_dependents();
  pdl_wait();  // the pool rows appended by the preceding launch, the plan, the previous merge
  const int n_items = a.direct ? a.n_tokens : a.header->n_items;
  const int total = n_items * a.kv_heads;

  for (int work = blockIdx.x; work < total; work += gridDim.x) {
    const int item = work / a.kv_heads, kvh = work - item * a.kv_heads;
    int token, kv_begin, kv_len, part;
    load_item(a, item, token, kv_begin, kv_len, part);
    const int* tbl = a.block_tables + __ldg(a.table_offset + __ldg(a.token_seq + token));
    const T* kc = static_cast<const T*>(a.k_cache) + kvh * D;
    const T* vc = static_cast<const T*>(a.v_cache) + kvh * D;

    // Query fragments: rows g and g+8 of the (padded) 16 x D group matrix.
    uint32_t qf[KS][4];
    {
      const T* qb = static_cast<const T*>(a.q) + (static_cast<size_t>(token) * a.q_heads + kvh * a.group) * D;
      const bool v0 = g < a.group, v1 = g + 8 < a.group;
      const uint32_t* q0 = reinterpret_cast<const uint32_t*>(qb + static_cast<size_t>(g) * D);
      const uint32_t* q1 = reinterpret_cast<const uint32_t*>(qb + static_cast<size_t>(g + 8) * D);
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        qf[s][0] = v0 ? __ldg(q0 + s * 8 + c) : 0u;
        qf[s][1] = v1 ? __ldg(q1 + s * 8 + c) : 0u;
        qf[s][2] = v0 ? __ldg(q0 + s * 8 + 4 + c) : 0u;
        qf[s][3] = v1 ? __ldg(q1 + s * 8 + 4 + c) : 0u;
      }
    }

    const int n_tiles = (kv_len + kTileKeys - 1) / kTileKeys;
    const int n_my = n_tiles > warp ? (n_tiles - warp + kDecodeWarps - 1) / kDecodeWarps : 0;

    // Issues the copies of this warp's i-th tile into ring stage i % STAGES.
    auto issue = [&](int i) {
      const int t = warp + i * kDecodeWarps;
      const uint32_t st = warp_smem + (i % STAGES) * S::kStageBytes;
      const int chunk = lane % CH, r0 = lane / CH;
#pragma unroll
      for (int p = 0; p < PASSES; ++p) {
        const int r = r0 + p * ROWS_PER_PASS;
        const int rel = t * kTileKeys + r;
        const bool valid = rel < kv_len;
        int64_t off = 0;
        if (valid) off = slot_of(tbl, kv_begin + rel, a.block_size, a.bs_log2) * kv_dim + chunk * 8;
        const uint32_t dst = st + r * S::kRowBytes + ((chunk ^ (r & 7)) << 4);
        cp_async16(dst, kc + off, valid ? 16 : 0);
        cp_async16(dst + S::kTileBytes, vc + off, valid ? 16 : 0);
      }
    };

    float o[2 * KS][4];
#pragma unroll
    for (int n = 0; n < 2 * KS; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
      if (i < n_my) issue(i);
      cp_async_commit();
    }

    for (int i = 0; i < n_my; ++i) {
      cp_async_wait<STAGES - 2>();
      __syncwarp();
      if (i + STAGES - 1 < n_my) issue(i + STAGES - 1);
      cp_async_commit();

      const uint32_t kst = warp_smem + (i % STAGES) * S::kStageBytes;
      const uint32_t vst = kst + S::kTileBytes;
      const int t = warp + i * kDecodeWarps;

      // S = Q K^T for 16 keys: two n-tiles of 8 keys.
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      {
        const int mi = lane >> 3, r = lane & 7;
        const int krow = ((mi >> 1) << 3) + r;
        const uint32_t rowaddr = kst + krow * S::kRowBytes;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int chunk = 2 * ks + (mi & 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(rowaddr + ((chunk ^ (krow & 7)) << 4), b0, b1, b2, b3);
          mma16816<T>(s[0], qf[ks], b0, b1);
          mma16816<T>(s[1], qf[ks], b2, b3);
        }
      }
      // Scale into the log2 domain and mask keys past the end of the item.
      const int col0 = t * kTileKeys + 2 * c;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = col0 + 8 * j + (e & 1);
          s[j][e] = col < kv_len ? s[j][e] * sl2 : -INFINITY;
        }
      }
      float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
      float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      // Every tile holds at least one valid key, so the new maxima are finite.
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float al0 = exp2f(m0 - mn0), al1 = exp2f(m1 - mn1);
      m0 = mn0;
      m1 = mn1;
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[j][0] = exp2f(s[j][0] - mn0);
        s[j][1] = exp2f(s[j][1] - mn0);
        s[j][2] = exp2f(s[j][2] - mn1);
        s[j][3] = exp2f(s[j][3] - mn1);
        ps0 += s[j][0] + s[j][1];
        ps1 += s[j][2] + s[j][3];
      }
      l0 = l0 * al0 + ps0;
      l1 = l1 * al1 + ps1;
#pragma unroll
      for (int n = 0; n < 2 * KS; ++n) {
        o[n][0] *= al0;
        o[n][1] *= al0;
        o[n][2] *= al1;
        o[n][3] *= al1;
      }
      // O += P V : P (16 heads x 16 keys) straight from the score registers.
      uint32_t pa[4];
      pa[0] = pack2<T>(s[0][0], s[0][1]);
      pa[1] = pack2<T>(s[0][2], s[0][3]);
      pa[2] = pack2<T>(s[1][0], s[1][1]);
      pa[3] = pack2<T>(s[1][2], s[1][3]);
      {
        const int mi = lane >> 3, r = lane & 7;
        const int vrow = ((mi & 1) << 3) + r;
        const uint32_t rowaddr = vst + vrow * S::kRowBytes;
#pragma unroll
        for (int np = 0; np < KS; ++np) {
          const int chunk = 2 * np + (mi >> 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(rowaddr + ((chunk ^ (vrow & 7)) << 4), b0, b1, b2, b3);
          mma16816<T>(o[2 * np], pa, b0, b1);
          mma16816<T>(o[2 * np + 1], pa, b2, b3);
        }
      }
    }
    cp_async_wait_all();
    // Row denominators: each lane of a quad summed a quarter of the keys.
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();  // every warp is done with its ring; reuse it for the merge

    float* sm_o = reinterpret_cast<float*>(smem_raw);
    float* sm_m = sm_o + kDecodeWarps * 16 * S::kLdo;
    float* sm_l = sm_m + kDecodeWarps * 16;
    float* sm_w = sm_l + kDecodeWarps * 16;
    if (c == 0) {
      sm_m[warp * 16 + g] = m0;
      sm_m[warp * 16 + g + 8] = m1;
      sm_l[warp * 16 + g] = l0;
      sm_l[warp * 16 + g + 8] = l1;
    }
#pragma unroll
    for (int n = 0; n < 2 * KS; ++n) {
      float* r0p = sm_o + (warp * 16 + g) * S::kLdo + n * 8 + 2 * c;
      float* r1p = sm_o + (warp * 16 + g + 8) * S::kLdo + n * 8 + 2 * c;
      *reinterpret_cast<float2*>(r0p) = make_float2(o[n][0], o[n][1]);
      *reinterpret_cast<float2*>(r1p) = make_float2(o[n][2], o[n][3]);
    }
    __syncthreads();
    merge_warps_and_store<T, true>(a, token, kvh * a.group, a.group, part, sm_m, sm_l, sm_o, S::kLdo, sm_w);
  }
}

// ============================================================================
// SIMT path: fp32 K/V (the 1e-5 parity configuration) and every geometry the
// tensor-core path does not take (head_dim not 64/128, group > 16, block sizes
// that are not powers of two).  head_dim <= 32 * DJ.
//
// Same work decomposition as above (a thread block per (token, key range) x kv head,
// the tiles of the range dealt to its four warps, the query heads of the group in
// batches of eight), fp32 arithmetic throughout.  Each warp streams tiles of KT keys
// through a private two-stage ring in shared memory: the K and V rows of a tile come
// in with 16-byte cp.async copies (gathered through the block table, rows padded by 16
// bytes against bank conflicts) while the previous tile is being used.  Scores: lane
// (h, k) computes q_h . K_k over the whole head dimension from shared memory with
// 16-byte reads, so a tile costs no shuffles for the dot products; the tile maximum and
// sum of a head take log2(KT) shuffles.  Output: lane d owns dims d, d + 32, ... of all
// eight heads and folds the tile's P V in from shared memory.
// ============================================================================
constexpr int kSimtHeadBatch = 8;

struct SimtLayout {
  int kt;            // keys per tile: 8, or 4 for rows beyond 512 bytes
  int row_bytes;     // one K or V row of one kv head, padded
  int stage_bytes;   // K tile then V tile
  int q_ld;          // floats per staged query row
  size_t off_o, off_m, off_l, off_w, off_p, off_ring, total;
};
template <typename T>
__host__ __device__ inline SimtLayout simt_layout(int D) {
  SimtLayout L;
  const int raw = D * static_cast<int>(sizeof(T));
  L.kt = raw <= 512 ? 8 : 4;
  L.row_bytes = ((raw + 15) & ~15) + 16;
  L.stage_bytes = 2 * L.kt * L.row_bytes;
  L.q_ld = ((D + 3) & ~3) + 4;
  size_t o = sizeof(float) * kSimtHeadBatch * L.q_ld;                 // sm_q
  L.off_o = o;  o += sizeof(float) * kDecodeWarps * 16 * (D + 1);      // sm_o
  L.off_m = o;  o += sizeof(float) * kDecodeWarps * 16;
  L.off_l = o;  o += sizeof(float) * kDecodeWarps * 16;
  L.off_w = o;  o += sizeof(float) * (kDecodeWarps + 2) * 16;
  L.off_p = o;  o += sizeof(float) * kDecodeWarps * (kSimtHeadBatch * 8 + kSimtHeadBatch);   // per warp: p[8][8], alpha[8]
  o = (o + 15) & ~static_cast<size_t>(15);
  L.off_ring = o;  o += static_cast<size_t>(kDecodeWarps) * 2 * L.stage_bytes;
  L.total = o;
  return L;
}

template <typename T> __device__ __forceinline__ void load_vec_f32(const unsigned char* p, float (&f)[16 / sizeof(T)]);
template <> __device__ __forceinline__ void load_vec_f32<float>(const unsigned char* p, float (&f)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load_vec_f32<__half>(const unsigned char* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 x = __half22float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
}
template <> __device__ __forceinline__ void load_vec_f32<__nv_bfloat16>(const unsigned char* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 x = __bfloat1622float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
}

template <typename T, int DJ>
__global__ void __launch_bounds__(kDecodeThreads) decode_simt_kernel(const DecodeArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int VE = 16 / static_cast<int>(sizeof(T));          // elements per 16-byte piece
  const int D = a.head_dim;
  const SimtLayout L = simt_layout<T>(D);
  const int KT = L.kt, ldo = D + 1;
  float* sm_q = reinterpret_cast<float*>(smem_raw);
  float* sm_o = reinterpret_cast<float*>(smem_raw + L.off_o);
  float* sm_m = reinterpret_cast<float*>(smem_raw + L.off_m);
  float* sm_l = reinterpret_cast<float*>(smem_raw + L.off_l);
  float* sm_w = reinterpret_cast<float*>(smem_raw + L.off_w);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* sm_p = reinterpret_cast<float*>(smem_raw + L.off_p) + warp * (kSimtHeadBatch * 8 + kSimtHeadBatch);   // [h][8]
  float* sm_alpha = sm_p + kSimtHeadBatch * 8;
  unsigned char* ring = smem_raw + L.off_ring + static_cast<size_t>(warp) * 2 * L.stage_bytes;
  const uint32_t ring_u32 = smem_u32(ring);
  const int kv_dim = a.kv_heads * D;
  const size_t pool_row_bytes = static_cast<size_t>(kv_dim) * sizeof(T);
  const int row_raw = D * static_cast<int>(sizeof(T));
  // 16-byte copies need rows that start and end on 16-byte boundaries in the pool
  const bool vec_ok = (row_raw & 15) == 0 && (pool_row_bytes & 15) == 0 &&
                      ((reinterpret_cast<uintptr_t>(a.k_cache) | reinterpret_cast<uintptr_t>(a.v_cache)) & 15) == 0;
  const int pieces = (row_raw + 15) >> 4;                       // 16-byte pieces per row

  pdl_launch_dependents();
  pdl_wait();
  const int n_items = a.direct ? a.n_tokens : a.header->n_items;
  const int total = n_items * a.kv_heads;

  for (int work = blockIdx.x; work < total; work += gridDim.x) {
    const int item = work / a.kv_heads, kvh = work - item * a.kv_heads;
    int token, kv_begin, kv_len, part;
    load_item(a, item, token, kv_begin, kv_len, part);
    const int* tbl = a.block_tables + __ldg(a.table_offset + __ldg(a.token_seq + token));
    const unsigned char* kc = static_cast<const unsigned char*>(a.k_cache) + static_cast<size_t>(kvh) * row_raw;
    const unsigned char* vc = static_cast<const unsigned char*>(a.v_cache) + static_cast<size_t>(kvh) * row_raw;
    const int n_tiles = (kv_len + KT - 1) / KT;
    const int n_my = n_tiles > warp ? (n_tiles - warp + kDecodeWarps - 1) / kDecodeWarps : 0;

    // Brings this warp's i-th tile into ring stage i & 1.  Rows past the end of the range are zero-filled.
    auto stage_tile = [&](int i) {
      const int t = warp + i * kDecodeWarps;
      unsigned char* st = ring + (i & 1) * L.stage_bytes;
      const uint32_t st_u32 = ring_u32 + (i & 1) * L.stage_bytes;
      for (int c = lane; c < KT * pieces; c += 32) {
        const int row = c / pieces, piece = c - row * pieces;
        const int rel = t * KT + row;
        const bool valid = rel < kv_len;
        size_t off = 0;
        if (valid) off = static_cast<size_t>(slot_of(tbl, kv_begin + rel, a.block_size, a.bs_log2)) * pool_row_bytes + piece * 16;
        const int dst = row * L.row_bytes + piece * 16;
        if (vec_ok) {
          cp_async16(st_u32 + dst, kc + off, valid ? 16 : 0);
          cp_async16(st_u32 + KT * L.row_bytes + dst, vc + off, valid ? 16 : 0);
        } else {
          // rows that are not 16-byte granular: element by element
          const int e0 = piece * VE;
          for (int e = 0; e < VE; ++e) {
            T kx = T(0), vx = T(0);
            if (valid && e0 + e < D) {
              kx = reinterpret_cast<const T*>(kc + static_cast<size_t>(slot_of(tbl, kv_begin + rel, a.block_size, a.bs_log2)) * pool_row_bytes)[e0 + e];
              vx = reinterpret_cast<const T*>(vc + static_cast<size_t>(slot_of(tbl, kv_begin + rel, a.block_size, a.bs_log2)) * pool_row_bytes)[e0 + e];
            }
            reinterpret_cast<T*>(st + dst)[e] = kx;
            reinterpret_cast<T*>(st + KT * L.row_bytes + dst)[e] = vx;
          }
        }
      }
    };

    for (int hb = 0; hb < a.group; hb += kSimtHeadBatch) {
      const int rows = min(kSimtHeadBatch, a.group - hb);
      const int head0 = kvh * a.group + hb;
      const T* qb = static_cast<const T*>(a.q) + (static_cast<size_t>(token) * a.q_heads + head0) * D;
      for (int i = threadIdx.x; i < kSimtHeadBatch * L.q_ld; i += kDecodeThreads) {
        const int h = i / L.q_ld, d = i - h * L.q_ld;
        sm_q[i] = (h < rows && d < D) ? Elem<T>::to_f32(qb[static_cast<size_t>(h) * D + d]) : 0.f;
      }
      __syncthreads();

      // this lane's (head, key) pairs of a tile: pair index lane and lane + 32, key = index % KT
      const int np = rows * KT;
      float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
      float acc[kSimtHeadBatch][DJ];
#pragma unroll
      for (int h = 0; h < kSimtHeadBatch; ++h)
#pragma unroll
        for (int j = 0; j < DJ; ++j) acc[h][j] = 0.f;

      if (n_my > 0) stage_tile(0);
      cp_async_commit();
      for (int i = 0; i < n_my; ++i) {
        if (i + 1 < n_my) stage_tile(i + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();
        const unsigned char* kst = ring + (i & 1) * L.stage_bytes;
        const unsigned char* vst = kst + KT * L.row_bytes;
        const int t = warp + i * kDecodeWarps;
        const int valid_keys = min(KT, kv_len - t * KT);
        // ---- scores and the tile's softmax weights ----
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const int idx = lane + 32 * s;
          const bool active = idx < np;
          const int k = idx % KT, h = active ? idx / KT : 0;
          float dot = 0.f;
          if (active) {
            const unsigned char* krow = kst + k * L.row_bytes;
            const float* qrow = sm_q + h * L.q_ld;
            for (int p = 0; p < pieces; ++p) {
              float kf[VE];
              load_vec_f32<T>(krow + p * 16, kf);
#pragma unroll
              for (int e = 0; e < VE; e += 4) {
                const float4 qv = *reinterpret_cast<const float4*>(qrow + p * VE + e);
                dot = fmaf(kf[e], qv.x, dot);
                dot = fmaf(kf[e + 1], qv.y, dot);
                dot = fmaf(kf[e + 2], qv.z, dot);
                dot = fmaf(kf[e + 3], qv.w, dot);
              }
            }
          }
          const float sc = (active && k < valid_keys) ? dot * a.scale : -INFINITY;
          float mx = sc;
          for (int o = 1; o < KT; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
          const float mn = fmaxf(m_run[s], mx);                       // finite for every active pair: key 0 of a tile is valid
          const float al = active ? expf(m_run[s] - mn) : 1.f;        // exp(-inf) = 0 on the first tile
          const float pw = active ? expf(sc - mn) : 0.f;
          float ps = pw;
          for (int o = 1; o < KT; o <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
          l_run[s] = l_run[s] * al + ps;
          m_run[s] = mn;
          if (active) {
            sm_p[h * 8 + k] = pw;
            if (k == 0) sm_alpha[h] = al;
          }
        }
        __syncwarp();
        // ---- O = O * alpha + P V, dims lane, lane + 32, ... of every head ----
        float vv[8][DJ];
#pragma unroll
        for (int k = 0; k < 8; ++k)
#pragma unroll
          for (int j = 0; j < DJ; ++j) {
            const int d = lane + 32 * j;
            vv[k][j] = (k < KT && d < D) ? Elem<T>::to_f32(reinterpret_cast<const T*>(vst + k * L.row_bytes)[d]) : 0.f;
          }
#pragma unroll
        for (int h = 0; h < kSimtHeadBatch; ++h) {
          if (h < rows) {
            const float al = sm_alpha[h];
            const float4 p0 = *reinterpret_cast<const float4*>(sm_p + h * 8);
            const float4 p1 = *reinterpret_cast<const float4*>(sm_p + h * 8 + 4);
            const float pk[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
            for (int j = 0; j < DJ; ++j) {
              float o = acc[h][j] * al;
#pragma unroll
              for (int k = 0; k < 8; ++k) o = fmaf(k < KT ? pk[k] : 0.f, vv[k][j], o);
              acc[h][j] = o;
            }
          }
        }
        __syncwarp();   // sm_p, sm_alpha and the stage are free for the next tile
      }
      cp_async_wait_all();
      // ---- this warp's partial state for the block-wide merge ----
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const int idx = lane + 32 * s;
        if (idx < np && idx % KT == 0) {
          sm_m[warp * 16 + idx / KT] = m_run[s];
          sm_l[warp * 16 + idx / KT] = l_run[s];
        }
      }
#pragma unroll
      for (int h = 0; h < kSimtHeadBatch; ++h) {
        if (h < rows) {
#pragma unroll
          for (int j = 0; j < DJ; ++j) {
            const int d = lane + 32 * j;
            if (d < D) sm_o[(warp * 16 + h) * ldo + d] = acc[h][j];
          }
        }
      }
      __syncthreads();
      merge_warps_and_store<T, false>(a, token, head0, rows, part, sm_m, sm_l, sm_o, ldo, sm_w);
    }
  }
}

template <typename T>
inline size_t simt_smem_bytes(int head_dim) { return simt_layout<T>(head_dim).total; }

}  // namespace pkv
