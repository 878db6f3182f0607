// Device-side step-index build: entry point pkv_step_pack_device of include/pkv.h.
//
// llm-engine rebuilds the step's index arrays on the host every step and sends them
// with six synchronous copies (CudaModel::upload_step_indices,
// src/model/cuda/cuda_model.cu:453-491; the loop over `seen` there is O(N*S)).  Here
// every sequence's block table stays resident on the device in a row of a table
// store; the host sends only what changed (blocks that were appended or rows that
// were released) and the step's slices (row, first position, length), and one block
// of threads writes positions, token_seq, slots, the concatenated tables and
// table_offset exactly as the host routine pkv_step_pack does for the same tokens:
// sequences numbered by first appearance, each distinct sequence's table appended
// once, slot = table[pos / bs] * bs + pos % bs (BlockTable::slot,
// include/engine/kv_cache.h:33-38).
#include <cstdint>

#include "launch_util.hpp"
#include "status.hpp"

namespace pkv {
namespace {

constexpr int kThreads = 1024;
constexpr int kMaxSlices = 4096;
constexpr int kPerThread = kMaxSlices / kThreads;

enum : int { kStTablesCap = 1, kStTokensCap = 2, kStPosBeyondTable = 4, kStBadRow = 8 };

struct StepPackArgs {
  const int32_t* updates;   // [n_updates][3] = row, block index (or -1: release the row), block id
  int n_updates;
  const int32_t* slices;    // [n_slices][3] = row, first position, length
  int n_slices;
  int32_t* seq_tables;      // [max_rows][table_stride]
  int32_t* seq_nblocks;     // [max_rows]
  int max_rows, table_stride;
  int block_size;
  int32_t* slots;
  int32_t* token_seq;
  int32_t* positions;
  int tokens_cap;
  int32_t* tables;
  int tables_cap;
  int32_t* table_offset;    // [n_slices] at most
  int32_t* counts;          // [4] = n_tokens, n_seqs, n_table, status bits
};

// Exclusive scan of three values per item over up to kMaxSlices items held kPerThread per thread.
__device__ __forceinline__ void block_scan3(int (&a)[kPerThread], int (&b)[kPerThread], int (&c)[kPerThread], int (&tot)[3],
                                            int (*warp_tot)[3]) {
  int sa = 0, sb = 0, sc = 0;
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    const int ta = a[i], tb = b[i], tc = c[i];
    a[i] = sa; b[i] = sb; c[i] = sc;
    sa += ta; sb += tb; sc += tc;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int ia = sa, ib = sb, ic = sc;   // inclusive over the warp
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int ua = __shfl_up_sync(0xffffffffu, ia, off), ub = __shfl_up_sync(0xffffffffu, ib, off),
              uc = __shfl_up_sync(0xffffffffu, ic, off);
    if (lane >= off) { ia += ua; ib += ub; ic += uc; }
  }
  if (lane == 31) { warp_tot[warp][0] = ia; warp_tot[warp][1] = ib; warp_tot[warp][2] = ic; }
  __syncthreads();
  if (warp == 0) {
    int wa = warp_tot[lane][0], wb = warp_tot[lane][1], wc = warp_tot[lane][2];
    int xa = wa, xb = wb, xc = wc;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int ua = __shfl_up_sync(0xffffffffu, xa, off), ub = __shfl_up_sync(0xffffffffu, xb, off),
                uc = __shfl_up_sync(0xffffffffu, xc, off);
      if (lane >= off) { xa += ua; xb += ub; xc += uc; }
    }
    warp_tot[lane][0] = xa - wa; warp_tot[lane][1] = xb - wb; warp_tot[lane][2] = xc - wc;   // exclusive
    if (lane == 31) { warp_tot[32][0] = xa; warp_tot[32][1] = xb; warp_tot[32][2] = xc; }
  }
  __syncthreads();
  const int oa = warp_tot[warp][0] + ia - sa, ob = warp_tot[warp][1] + ib - sb, oc = warp_tot[warp][2] + ic - sc;
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) { a[i] += oa; b[i] += ob; c[i] += oc; }
  tot[0] = warp_tot[32][0]; tot[1] = warp_tot[32][1]; tot[2] = warp_tot[32][2];
}

__global__ void __launch_bounds__(kThreads, 1) step_pack_kernel(const StepPackArgs a) {
  extern __shared__ int32_t sm[];
  int32_t* s_row = sm;                        // [kMaxSlices] row of slice i (-1: invalid)
  int32_t* s_tok = sm + kMaxSlices;           // first packed token of slice i
  int32_t* s_idx = sm + 2 * kMaxSlices;       // step-local sequence number of slice i
  int32_t* s_off = sm + 3 * kMaxSlices;       // where its table starts in `tables` (of its first appearance)
  __shared__ int warp_tot[33][3];
  __shared__ int s_status;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_status = 0;
  // No early release of the dependents: the kernels behind this one read the arrays it writes before
  // their own griddepcontrol.wait (they treat the step's index arrays as complete from the start).
  pdl_wait();

  // ---- 0. bring the resident tables up to date: releases first, then appended blocks ----
  for (int u = tid; u < a.n_updates; u += kThreads) {
    const int row = a.updates[3 * u], idx = a.updates[3 * u + 1];
    if (row < 0 || row >= a.max_rows) { atomicOr(&s_status, kStBadRow); continue; }
    if (idx < 0) a.seq_nblocks[row] = 0;
  }
  __syncthreads();
  for (int u = tid; u < a.n_updates; u += kThreads) {
    const int row = a.updates[3 * u], idx = a.updates[3 * u + 1], blk = a.updates[3 * u + 2];
    if (row < 0 || row >= a.max_rows || idx < 0) continue;
    if (idx >= a.table_stride) { atomicOr(&s_status, kStBadRow); continue; }
    a.seq_tables[static_cast<size_t>(row) * a.table_stride + idx] = blk;
    atomicMax(&a.seq_nblocks[row], idx + 1);
  }
  __threadfence_block();
  __syncthreads();

  // ---- 1. slices -> shared memory ----
  for (int i = tid; i < a.n_slices; i += kThreads) {
    int row = a.slices[3 * i];
    if (row < 0 || row >= a.max_rows) { atomicOr(&s_status, kStBadRow); row = -1; }
    s_row[i] = row;
  }
  __syncthreads();

  // ---- 2. first appearance of each slice's sequence, then three exclusive scans ----
  int v_len[kPerThread], v_uniq[kPerThread], v_nb[kPerThread], first[kPerThread];
#pragma unroll
  for (int k = 0; k < kPerThread; ++k) {
    const int i = tid * kPerThread + k;
    v_len[k] = v_uniq[k] = v_nb[k] = 0;
    first[k] = i;
    if (i < a.n_slices && s_row[i] >= 0) {
      const int row = s_row[i];
      for (int j = 0; j < i; ++j)
        if (s_row[j] == row) { first[k] = j; break; }
      v_len[k] = max(a.slices[3 * i + 2], 0);
      if (first[k] == i) {
        v_uniq[k] = 1;
        v_nb[k] = a.seq_nblocks[row];
      }
    }
  }
  int tot[3];
  block_scan3(v_len, v_uniq, v_nb, tot, warp_tot);
#pragma unroll
  for (int k = 0; k < kPerThread; ++k) {
    const int i = tid * kPerThread + k;
    if (i < a.n_slices) {
      s_tok[i] = v_len[k];
      s_idx[i] = v_uniq[k];     // meaningful where the slice is a first appearance; fixed up below
      s_off[i] = v_nb[k];
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kPerThread; ++k) {
    const int i = tid * kPerThread + k;
    if (i < a.n_slices && first[k] != i) {   // a later slice of a sequence takes its first slice's number
      s_idx[i] = s_idx[first[k]];
      s_off[i] = s_off[first[k]];
    }
  }
  const int n_tokens = tot[0], n_seqs = tot[1], n_table = tot[2];
  if (n_tokens > a.tokens_cap) atomicOr(&s_status, kStTokensCap);
  if (n_table > a.tables_cap) atomicOr(&s_status, kStTablesCap);
  __syncthreads();
  const bool fits = n_tokens <= a.tokens_cap && n_table <= a.tables_cap;

  // ---- 3. outputs: a warp per slice ----
  if (fits) {
    for (int i = warp; i < a.n_slices; i += kThreads / 32) {
      const int row = s_row[i];
      if (row < 0) continue;
      const int start = a.slices[3 * i + 1], len = max(a.slices[3 * i + 2], 0);
      const int nb = a.seq_nblocks[row];
      const int32_t* tbl = a.seq_tables + static_cast<size_t>(row) * a.table_stride;
      const int base = s_tok[i], idx = s_idx[i], off = s_off[i];
      bool first_here = true;
      for (int j = 0; j < i; ++j)           // warp-uniform; S is small
        if (s_row[j] == row) { first_here = false; break; }
      if (first_here) {
        if (lane == 0) a.table_offset[idx] = off;
        for (int b = lane; b < nb; b += 32) a.tables[off + b] = tbl[b];
      }
      for (int t = lane; t < len; t += 32) {
        const int pos = start + t;
        const int bi = pos / a.block_size;
        int slot = 0;
        if (pos < 0 || bi >= nb) atomicOr(&s_status, kStPosBeyondTable);
        else slot = tbl[bi] * a.block_size + (pos - bi * a.block_size);
        a.positions[base + t] = pos;
        a.token_seq[base + t] = idx;
        a.slots[base + t] = slot;
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    a.counts[0] = n_tokens;
    a.counts[1] = n_seqs;
    a.counts[2] = n_table;
    a.counts[3] = s_status;
  }
}

}  // namespace
}  // namespace pkv

extern "C" int pkv_step_pack_device(const int32_t* d_updates, int n_updates, const int32_t* d_slices, int n_slices,
                                    int32_t* d_seq_tables, int32_t* d_seq_nblocks, int max_rows, int table_stride,
                                    int block_size, int32_t* d_slots, int32_t* d_token_seq, int32_t* d_positions,
                                    int tokens_cap, int32_t* d_tables, int tables_cap, int32_t* d_table_offset,
                                    int32_t* d_counts, pkv_stream stream) {
  using namespace pkv;
  const char* fn = "pkv_step_pack_device";
  if (n_updates < 0 || n_slices < 0 || max_rows <= 0 || table_stride <= 0 || block_size <= 0 || tokens_cap < 0 || tables_cap < 0)
    return fail(PKV_E_ARG, "%s: negative count or non-positive geometry", fn);
  if (n_slices > kMaxSlices) return fail(PKV_E_UNSUPPORTED, "%s: %d slices; at most %d per step", fn, n_slices, kMaxSlices);
  if (!d_seq_tables || !d_seq_nblocks || !d_counts || (n_updates > 0 && !d_updates) || (n_slices > 0 && !d_slices))
    return fail(PKV_E_ARG, "%s: null device pointer", fn);
  if (n_slices > 0 && (!d_slots || !d_token_seq || !d_positions || !d_tables || !d_table_offset))
    return fail(PKV_E_ARG, "%s: null output pointer", fn);
  StepPackArgs a;
  a.updates = d_updates; a.n_updates = n_updates;
  a.slices = d_slices; a.n_slices = n_slices;
  a.seq_tables = d_seq_tables; a.seq_nblocks = d_seq_nblocks;
  a.max_rows = max_rows; a.table_stride = table_stride; a.block_size = block_size;
  a.slots = d_slots; a.token_seq = d_token_seq; a.positions = d_positions; a.tokens_cap = tokens_cap;
  a.tables = d_tables; a.tables_cap = tables_cap; a.table_offset = d_table_offset; a.counts = d_counts;
  constexpr int smem = 4 * kMaxSlices * static_cast<int>(sizeof(int32_t));
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    const cudaError_t e = cudaFuncSetAttribute(step_pack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(PKV_E_CUDA, "%s: cannot reserve %d bytes of shared memory: %s", fn, smem, cudaGetErrorString(e));
    configured_device = dev;
  }
  launch_pdl(step_pack_kernel, dim3(1), dim3(kThreads), smem, static_cast<cudaStream_t>(stream), a);
  return check_launch("step_pack_kernel");
}
