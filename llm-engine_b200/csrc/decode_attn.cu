// C-ABI entry points for paged decode attention (include/pkv.h, "decode attention"):
// argument validation, split-K planning (host and device), kernel selection.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <type_traits>
#include <cstring>
#include <mutex>
#include <vector>

#include "decode_attn.cuh"
#include "decode_tma.cuh"
#include "launch_util.hpp"
#include "status.hpp"

// Scratch for pkv_decode_attn_bf16_builtin_scratch: lives in the library's own device
// image, one copy per GPU that loads it, for the life of the process.  In host code
// this name is only a handle for cudaGetSymbolAddress, never a usable pointer.
constexpr size_t kBuiltinScratchBytes = 32u << 20;
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

namespace pkv {
int prefill_read_flags(unsigned int* flags);  // prefill_attn.cu
template <typename T>
int prefill_launch(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                   const int* table_offset, const int* q_start, const int* q_len, const int* ctx_len, void* out,
                   int n_tokens, int n_seqs, int max_q_len, int q_heads, int kv_heads, int head_dim, int block_size,
                   int num_blocks, float scale, pkv_stream stream, const int* d_dims, bool may_allocate);
unsigned int* error_mirror(bool create);      // error_mirror.cu
unsigned int take_error_mirror();
int check_error_mirror(const char* fn);
namespace {

// ---- tuning knobs (read once) ---------------------------------------------------
struct Tuning {
  int target_ctas;   // thread blocks the planner aims for when it splits
  int wave_ctas;     // below this many blocks, smaller chunks are tried
  int forced_chunk;  // 0 = rule
  int variant;       // ring depth / occupancy variant of the tensor-core kernel
  int use_tma;       // 1: TMA + warp-specialised kernel where the geometry allows (default)
  int max_extra_cap;
  int cluster_max_keys;  // the cluster form of small steps is offered only while no warp would get more keys than this
  int cluster_size;      // 0 = as many blocks per cluster as stay resident; otherwise at most this many
};
int env_int(const char* name, int dflt) {
  const char* e = std::getenv(name);
  if (!e || !*e) return dflt;
  return std::atoi(e);
}
const Tuning& tuning() {
  static const Tuning t = [] {
    Tuning x;
    x.target_ctas = env_int("PKV_DECODE_TARGET_CTAS", 4736);
    x.wave_ctas = env_int("PKV_DECODE_WAVE_CTAS", 1776);  // workers (warps) resident on a 148-SM part
    x.forced_chunk = env_int("PKV_DECODE_CHUNK", 0);
    x.variant = env_int("PKV_DECODE_VARIANT", 0);
    x.use_tma = env_int("PKV_DECODE_TMA", 1);
    x.max_extra_cap = 16384;
    x.cluster_max_keys = env_int("PKV_DECODE_CLUSTER_MAX_KEYS", 256);
    x.cluster_size = env_int("PKV_DECODE_CLUSTER_SIZE", 0);
    return x;
  }();
  return t;
}

// PKV_DECODE_CLUSTER=0: the host planner never chooses the cluster form of the attention launch for small
// steps (read at every planning call, so a process can switch it).  On by default: on the step it is
// meant for (64 sequences, 256-2,048 keys) a layer takes 10.3 us against 12.3 us for the two ordinary
// launches inside a replayed graph, and a fifth less time launched eagerly.
bool cluster_form_enabled() {
  const char* e = std::getenv("PKV_DECODE_CLUSTER");
  return !(e && e[0] == '0');
}

int max_extra(int kv_heads) { return (tuning().max_extra_cap + kv_heads - 1) / kv_heads; }

// ---- device planner ---------------------------------------------------------------
// One block builds the whole work list from the device copy of token_pos.
constexpr int kPlanThreads = 1024;

// Mixed-step routing (optional first phase of the planner).  llm-engine's forward pass sends a
// whole step through one attention call: prefill slices first, then decode tokens, a slice's tokens
// packed consecutively (src/model/cuda/cuda_model.cu:362-377, 434-447; include/engine/sequence.h:74-89).
// A run is a maximal stretch of packed tokens of one sequence at consecutive positions.  Runs of at
// least min_run tokens are prefill chunks: they get a (first row, length, cached context, table
// offset) record for the tensor-core prefill kernel and their tokens an effective length of 0,
// which takes them out of the decode plan; every other token keeps position + 1.
struct RouteArgs {
  const int* token_seq;
  const int* table_offset;
  int min_run, q_heads;
  int* run_start;   // [n_tokens] scratch: first token of the run a token belongs to
  int* run_len;     // [n_tokens] scratch: length of a run, stored at its first token
  int* eff_len;     // [n_tokens] out
  int* q_start;     // [n_tokens / min_run + 1] out, and the three below
  int* q_len;
  int* ctx_len;
  int* tbl_off;
  int* dims;        // [4] out: runs, 128-row tiles of the longest run, prefill work items, decode tokens
};

__device__ void route_phase(const int* __restrict__ token_pos, int n, const RouteArgs& r, int* sm_scan, int* sm_misc) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto is_start = [&](int t) {
    return t == 0 || r.token_seq[t] != r.token_seq[t - 1] || token_pos[t] != token_pos[t - 1] + 1;
  };
  // 1. running maximum of the start indices = first token of each token's run
  int carry = 0;
  for (int base = 0; base < n; base += kPlanThreads) {
    const int t = base + tid;
    int v = (t < n && is_start(t)) ? t : -1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v = max(v, x);
    }
    if (lane == 31) sm_scan[warp] = v;
    __syncthreads();
    if (warp == 0) {
      int a = sm_scan[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int x = __shfl_up_sync(0xffffffffu, a, o);
        if (lane >= o) a = max(a, x);
      }
      sm_scan[lane] = a;
    }
    __syncthreads();
    v = max(v, max(warp ? sm_scan[warp - 1] : -1, carry));
    if (t < n) r.run_start[t] = v;
    carry = max(carry, sm_scan[kPlanThreads / 32 - 1]);
    __syncthreads();
  }
  // 2. the last token of a run stores the run's length at its first token
  for (int t = tid; t < n; t += kPlanThreads) {
    if (t == n - 1 || is_start(t + 1)) {
      const int rs = r.run_start[t];
      r.run_len[rs] = t - rs + 1;
    }
  }
  if (tid == 0) { sm_misc[0] = 0; sm_misc[1] = 0; sm_misc[2] = 0; }   // runs so far, longest run, decode tokens
  __syncthreads();
  // 3. effective lengths and the records of the long runs, in packed order
  for (int base = 0; base < n; base += kPlanThreads) {
    const int t = base + tid;
    int flag = 0, len = 0;
    if (t < n) {
      const int rs = r.run_start[t];
      len = r.run_len[rs];
      const bool long_run = len >= r.min_run;
      r.eff_len[t] = long_run ? 0 : max(token_pos[t], 0) + 1;
      flag = (long_run && rs == t) ? 1 : 0;
      if (!long_run) atomicAdd(&sm_misc[2], 1);
    }
    int sc = flag;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, sc, o);
      if (lane >= o) sc += x;
    }
    if (lane == 31) sm_scan[warp] = sc;
    __syncthreads();
    if (warp == 0) {
      int a = sm_scan[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int x = __shfl_up_sync(0xffffffffu, a, o);
        if (lane >= o) a += x;
      }
      sm_scan[lane] = a;
    }
    __syncthreads();
    if (flag) {
      const int i = sm_misc[0] + (warp ? sm_scan[warp - 1] : 0) + sc - 1;
      r.q_start[i] = t;
      r.q_len[i] = len;
      r.ctx_len[i] = max(token_pos[t], 0);
      r.tbl_off[i] = r.table_offset[r.token_seq[t]];
      atomicMax(&sm_misc[1], len);
    }
    __syncthreads();
    if (tid == 0) sm_misc[0] += sm_scan[kPlanThreads / 32 - 1];
    __syncthreads();
  }
  if (tid == 0) {
    const int tiles = (sm_misc[1] + 127) / 128;
    r.dims[0] = sm_misc[0];
    r.dims[1] = tiles;
    r.dims[2] = sm_misc[0] * tiles * r.q_heads;
    r.dims[3] = sm_misc[2];
  }
  __syncthreads();
}

template <bool ROUTE>
__global__ void __launch_bounds__(kPlanThreads) decode_plan_kernel(const int* __restrict__ token_pos, int n_tokens,
                                                                    int kv_heads, long long extra_budget,
                                                                    int wave_ctas, int forced_chunk,
                                                                    PlanHeader* header, TokSplit* tok_split,
                                                                    int* counters, WorkItem* items, const RouteArgs route) {
  __shared__ unsigned long long sm_items[kNumChunkCandidates];
  __shared__ int sm_chunk;
  __shared__ int sm_scan_items[kPlanThreads / 32], sm_scan_parts[kPlanThreads / 32];
  __shared__ int sm_carry_items, sm_carry_parts;
  __shared__ int sm_misc[4];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if constexpr (ROUTE) route_phase(token_pos, n_tokens, route, sm_scan_items, sm_misc);
  // keys the decode path handles for token t: position + 1, or 0 for a token the router gave to the prefill kernel
  auto length_of = [&](int t) {
    if constexpr (ROUTE) return route.eff_len[t];
    return max(token_pos[t], 0) + 1;
  };
  if (tid < kNumChunkCandidates) sm_items[tid] = 0ull;
  if (tid == 0) { sm_carry_items = 0; sm_carry_parts = 0; }
  __syncthreads();
  {
    unsigned long long loc[kNumChunkCandidates];
#pragma unroll
    for (int j = 0; j < kNumChunkCandidates; ++j) loc[j] = 0ull;
    for (int t = tid; t < n_tokens; t += kPlanThreads) {
      const int L = length_of(t);
#pragma unroll
      for (int j = 0; j < kNumChunkCandidates; ++j) loc[j] += static_cast<unsigned>((L + (kMinChunk << j) - 1) / (kMinChunk << j));
    }
#pragma unroll
    for (int j = 0; j < kNumChunkCandidates; ++j) {
      unsigned long long v = loc[j];
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && v) atomicAdd(&sm_items[j], v);
    }
  }
  __syncthreads();
  if (tid == 0) {
    long long items_at[kNumChunkCandidates];
    for (int j = 0; j < kNumChunkCandidates; ++j) items_at[j] = static_cast<long long>(sm_items[j]);
    sm_chunk = choose_chunk(items_at, n_tokens, kv_heads, extra_budget, wave_ctas, forced_chunk);
  }
  __syncthreads();
  const int chunk = sm_chunk;

  for (int base = 0; base < n_tokens; base += kPlanThreads) {
    const int t = base + tid;
    int L = 0, ns = 0;
    if (t < n_tokens) {
      L = length_of(t);
      ns = L == 0 ? 0 : (chunk > 0 ? (L + chunk - 1) / chunk : 1);
    }
    const int np = ns > 1 ? ns : 0;
    // inclusive scans of ns and np across the block
    int si = ns, sp = np;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, si, o), b = __shfl_up_sync(0xffffffffu, sp, o);
      if (lane >= o) { si += a; sp += b; }
    }
    if (lane == 31) { sm_scan_items[warp] = si; sm_scan_parts[warp] = sp; }
    __syncthreads();
    if (warp == 0) {
      int a = sm_scan_items[lane], b = sm_scan_parts[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int x = __shfl_up_sync(0xffffffffu, a, o), y = __shfl_up_sync(0xffffffffu, b, o);
        if (lane >= o) { a += x; b += y; }
      }
      sm_scan_items[lane] = a;
      sm_scan_parts[lane] = b;
    }
    __syncthreads();
    const int item0 = sm_carry_items + (warp ? sm_scan_items[warp - 1] : 0) + si - ns;
    const int part0 = sm_carry_parts + (warp ? sm_scan_parts[warp - 1] : 0) + sp - np;
    if (t < n_tokens) {
      tok_split[t] = TokSplit{part0, ns};
      for (int s = 0; s < ns; ++s) {
        const int b = chunk > 0 ? s * chunk : 0;
        const int len = chunk > 0 ? min(chunk, L - b) : L;
        items[item0 + s] = WorkItem{t, b, len, ns > 1 ? part0 + s : -1};
      }
    }
    __syncthreads();
    if (tid == 0) {
      sm_carry_items += sm_scan_items[kPlanThreads / 32 - 1];
      sm_carry_parts += sm_scan_parts[kPlanThreads / 32 - 1];
    }
    __syncthreads();
  }
  for (int i = tid; i < n_tokens * kv_heads; i += kPlanThreads) counters[i] = 0;
  if (tid == 0) {
    header->magic = kPlanMagic;
    header->n_items = sm_carry_items;
    header->chunk = chunk;
    header->n_tokens = n_tokens;
    header->n_parts = sm_carry_parts;
    header->kv_heads = kv_heads;
    header->pad[0] = header->pad[1] = 0;
  }
}

// ---- kernel launch ----------------------------------------------------------------
template <typename T> struct IsF32 { static constexpr bool value = false; };
template <> struct IsF32<float> { static constexpr bool value = true; };

template <typename T, int D, int STAGES, int MINB>
int launch_mma(const DecodeArgs& a, int grid, cudaStream_t stream) {
  using S = MmaSmem<D, STAGES>;
  auto kern = decode_mma_kernel<T, D, STAGES, MINB>;
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
    if (e != cudaSuccess) return fail(PKV_E_CUDA, "decode: cannot reserve %d bytes of shared memory: %s", S::kBytes, cudaGetErrorString(e));
    configured_device = dev;
  }
  launch_pdl(kern, dim3(grid), dim3(kDecodeThreads), S::kBytes, stream, a);
  return check_launch("decode_mma_kernel");
}

int persistent_sms() {
  static thread_local int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

template <typename T, int D, int NT, int MT, int NSTAGES, int WARPS, int MINB, int TOK = 1, bool FUSED = false>
int launch_tma(const DecodeArgs& a, int grid, cudaStream_t stream) {
  if constexpr (TOK == 1 && !FUSED) {
    if (a.new_k != nullptr) return launch_tma<T, D, NT, MT, NSTAGES, WARPS, MINB, 1, true>(a, grid, stream);
  }
  using S = TmaSmem<D, MT, NSTAGES, WARPS>;
  auto kern = decode_tma_kernel<T, D, NT, MT, NSTAGES, WARPS, MINB, TOK, FUSED>;
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
    if (e != cudaSuccess) return fail(PKV_E_CUDA, "decode: cannot reserve %d bytes of shared memory: %s", S::kBytes, cudaGetErrorString(e));
    configured_device = dev;
  }
  alignas(64) CUtensorMap kmap, vmap;
  constexpr bool is_bf16 = !std::is_same<T, __half>::value;
  const int kv_dim = a.kv_heads * a.head_dim;
  int st = make_pool_tensor_map(&kmap, a.k_cache, is_bf16, kv_dim, 16, a.pool_rows);
  if (st != PKV_OK) return st;
  st = make_pool_tensor_map(&vmap, a.v_cache, is_bf16, kv_dim, 16, a.pool_rows);
  if (st != PKV_OK) return st;
  // `grid` counts work units; every warp is a worker and blocks are persistent:
  // as many as can be resident, each warp striding through the unit list.
  int blocks = (grid + WARPS - 1) / WARPS;
  const int resident = persistent_sms() * MINB;
  if (blocks > resident) blocks = resident;
  launch_pdl(kern, dim3(blocks), dim3(WARPS * 32), S::kBytes, stream, a, kmap, vmap);
  return check_launch("decode_tma_kernel");
}

std::atomic<unsigned long long> g_cluster_launches{0};   // pkv_debug_cluster_launches

// Small steps as thread-block clusters (decode_tma_kernel with CLUSTER): one cluster of `cs` blocks
// per (token, kv head), merge inside the launch.  *launched stays false, with nothing enqueued, when
// this device cannot hold all the clusters at once (they would queue behind one another): the
// caller then takes the ordinary path.
template <typename T, bool FUSED>
int launch_tma_cluster_impl(const DecodeArgs& a, int cs, cudaStream_t stream, bool* launched) {
  constexpr int WARPS = 4;
  using S = TmaSmem<64, 2, 2, WARPS>;
  auto kern = decode_tma_kernel<T, 64, 1, 2, 2, WARPS, 3, 1, FUSED, true>;
  *launched = false;
  const long long pairs = static_cast<long long>(a.n_tokens) * a.kv_heads;
  if (!cluster_size_ok(cs) || pairs * cs > 0x7fffffffll) return PKV_OK;
  constexpr int kSmem = S::kBytes + kClusterLandBytes;
  static thread_local int configured_device = -1;
  static thread_local int max_clusters[9];
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return fail(PKV_E_CUDA, "decode: cannot reserve %d bytes of shared memory: %s", kSmem, cudaGetErrorString(e));
    for (int i = 0; i < 9; ++i) max_clusters[i] = -1;
    configured_device = dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(pairs * cs));
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(cs);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  if (max_clusters[cs] < 0) {
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    max_clusters[cs] = n;
  }
  if (pairs > max_clusters[cs]) return PKV_OK;
  alignas(64) CUtensorMap kmap, vmap;
  constexpr bool is_bf16 = !std::is_same<T, __half>::value;
  const int kv_dim = a.kv_heads * a.head_dim;
  int st = make_pool_tensor_map(&kmap, a.k_cache, is_bf16, kv_dim, 16, a.pool_rows);
  if (st != PKV_OK) return st;
  st = make_pool_tensor_map(&vmap, a.v_cache, is_bf16, kv_dim, 16, a.pool_rows);
  if (st != PKV_OK) return st;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, kern, a, kmap, vmap);
  *launched = true;
  g_cluster_launches.fetch_add(1, std::memory_order_relaxed);
  return check_launch("decode_tma_kernel (clusters)");
}

template <typename T>
int launch_tma_cluster(const DecodeArgs& a, int cs, cudaStream_t stream, bool* launched) {
  *launched = false;
  if constexpr (IsF32<T>::value) {
    return PKV_OK;
  } else {
    if (a.new_k != nullptr) return launch_tma_cluster_impl<T, true>(a, cs, stream, launched);
    return launch_tma_cluster_impl<T, false>(a, cs, stream, launched);
  }
}

template <typename T, int DJ>
int launch_simt(const DecodeArgs& a, int grid, cudaStream_t stream) {
  const size_t smem = simt_smem_bytes<T>(a.head_dim);
  auto kern = decode_simt_kernel<T, DJ>;
  if (smem > 48 * 1024) {
    static thread_local int configured_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_device != dev) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      if (e != cudaSuccess) return fail(PKV_E_CUDA, "decode: cannot reserve shared memory: %s", cudaGetErrorString(e));
      configured_device = dev;
    }
  }
  launch_pdl(kern, dim3(grid), dim3(kDecodeThreads), smem, stream, a);
  return check_launch("decode_simt_kernel");
}

template <typename T, bool LOG2>
int launch_combine(const DecodeArgs& a, cudaStream_t stream) {
  if (a.direct) return PKV_OK;
  long long blocks = static_cast<long long>(a.n_tokens) * a.kv_heads;
  const long long cap = static_cast<long long>(persistent_sms()) * 16;
  if (blocks > cap) blocks = cap;
  launch_pdl(decode_combine_kernel<T, LOG2>, dim3(static_cast<unsigned>(blocks)), dim3(kCombineThreads), 0, stream, a);
  return check_launch("decode_combine_kernel");
}

// Whether this geometry runs on decode_tma_kernel.
template <typename T>
bool tma_path(const DecodeArgs& a) {
  if constexpr (IsF32<T>::value) return false;
  return (a.head_dim == 64 || a.head_dim == 128) && a.group <= 16 && a.bs_log2 >= 4 && a.scale > 0.f && tuning().use_tma &&
         tensor_map_encoder() != nullptr;
}

template <typename T>
int launch_decode_main(const DecodeArgs& a, int grid, cudaStream_t stream, bool* log2_domain) {
  *log2_domain = true;
  if constexpr (!IsF32<T>::value) {
    const bool mma_ok = (a.head_dim == 64 || a.head_dim == 128) && a.group <= 16 && a.bs_log2 >= 0;
    const bool tma_ok = tma_path<T>(a);
    if (tma_ok) {
      const int variant = tuning().variant;
      if (a.head_dim == 64) {
        if (a.group <= 8) {
          // <T, head_dim, head tiles, 16-key tiles per stage, stages per warp, warps, blocks per SM>
          if (variant == 1) return launch_tma<T, 64, 1, 1, 3, 4, 4>(a, grid, stream);
          if (variant == 2) return launch_tma<T, 64, 1, 1, 4, 4, 3>(a, grid, stream);
          if (variant == 3) return launch_tma<T, 64, 1, 2, 3, 4, 2>(a, grid, stream);
          if (variant == 4) return launch_tma<T, 64, 1, 2, 2, 6, 2>(a, grid, stream);
          if (variant == 5) return launch_tma<T, 64, 1, 2, 2, 7, 2>(a, grid, stream);
          return launch_tma<T, 64, 1, 2, 2, 4, 3>(a, grid, stream);  // measured best on B200
        }
        return launch_tma<T, 64, 2, 1, 4, 4, 3>(a, grid, stream);
      }
      if (a.group <= 8) return launch_tma<T, 128, 1, 1, 3, 4, 2>(a, grid, stream);
      return launch_tma<T, 128, 2, 1, 3, 4, 2>(a, grid, stream);
    }
    if (mma_ok) {
      const int variant = tuning().variant;
      if (a.head_dim == 64) {
        if (variant == 1) return launch_mma<T, 64, 3, 4>(a, grid, stream);
        if (variant == 2) return launch_mma<T, 64, 6, 2>(a, grid, stream);
        return launch_mma<T, 64, 4, 3>(a, grid, stream);
      }
      return launch_mma<T, 128, 3, 2>(a, grid, stream);
    }
  }
  *log2_domain = false;
  const int dj = (a.head_dim + 31) / 32;
  if (dj <= 2) return launch_simt<T, 2>(a, grid, stream);
  if (dj <= 4) return launch_simt<T, 4>(a, grid, stream);
  return launch_simt<T, 8>(a, grid, stream);
}

// Whether the geometry runs on the TMA kernel (the only one that takes shared-prefix units).
template <typename T>
bool shared_units_ok(const DecodeArgs& a) {
  if constexpr (IsF32<T>::value) return false;
  return a.head_dim == 64 && a.group <= 8 && a.bs_log2 >= 4 && a.scale > 0.f && tuning().use_tma && tensor_map_encoder() != nullptr;
}

// Shared-prefix units first (one K/V fetch for up to four tokens), then the attention kernel
// over the ordinary items, then (when the plan split any token) the merge of the partials.
template <typename T>
int launch_decode(const DecodeArgs& a, int grid, cudaStream_t stream, bool has_splits) {
  bool log2_domain = true;
  if constexpr (!IsF32<T>::value) {
    if (a.n_shared > 0) {
      long long units = static_cast<long long>(a.n_shared) * a.kv_heads;
      if (units > 0x7fffffffll) units = 0x7fffffffll;
      // <T, head_dim, head tiles (4 tokens x 1), 16-key tiles per stage, stages, warps, blocks per SM, tokens per unit>
      const int st = launch_tma<T, 64, 4, 2, 2, 4, 2, 4>(a, static_cast<int>(units), stream);
      if (st != PKV_OK) return st;
    }
  }
  const int st = launch_decode_main<T>(a, grid, stream, &log2_domain);
  if (st != PKV_OK || (!has_splits && a.n_peers == 0)) return st;   // with peers the merge kernel also does the exchange
  return log2_domain ? launch_combine<T, true>(a, stream) : launch_combine<T, false>(a, stream);
}

int validate_geometry(const char* fn, int n_tokens, int q_heads, int kv_heads, int head_dim, int block_size) {
  if (q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || block_size <= 0)
    return fail(PKV_E_ARG, "%s: q_heads %d, kv_heads %d, head_dim %d, block_size %d must all be > 0", fn, q_heads, kv_heads, head_dim, block_size);
  if (q_heads % kv_heads != 0)
    return fail(PKV_E_UNSUPPORTED, "%s: q_heads %d is not a multiple of kv_heads %d", fn, q_heads, kv_heads);
  if (head_dim > 256)
    return fail(PKV_E_UNSUPPORTED, "%s: head_dim %d exceeds 256, the largest the accumulators cover", fn, head_dim);
  (void)n_tokens;
  return PKV_OK;
}

int validate_pointers(const char* fn, const void* q, const void* kc, const void* vc, const int* bt, const int* to,
                      const int* ts, const int* tp, const void* out, size_t row_bytes) {
  if (!q || !kc || !vc || !bt || !to || !ts || !tp || !out) return fail(PKV_E_ARG, "%s: null device pointer", fn);
  if (row_bytes % 16 == 0 &&
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc) |
        reinterpret_cast<uintptr_t>(out)) & 15))
    return fail(PKV_E_ARG, "%s: q, out and the K/V pools must be 16-byte aligned", fn);
  return PKV_OK;
}

int log2_exact(int x) {
  if (x <= 0 || (x & (x - 1))) return -1;
  int l = 0;
  while ((1 << l) < x) ++l;
  return l;
}

void fill_args(DecodeArgs& a, const void* q, const void* kc, const void* vc, const int* bt, const int* to,
               const int* ts, const int* tp, void* out, int n_tokens, int q_heads, int kv_heads, int head_dim,
               int block_size, float scale) {
  a.q = q; a.k_cache = kc; a.v_cache = vc;
  a.block_tables = bt; a.table_offset = to; a.token_seq = ts; a.token_pos = tp;
  a.out = out;
  a.n_tokens = n_tokens; a.q_heads = q_heads; a.kv_heads = kv_heads; a.head_dim = head_dim;
  a.group = q_heads / kv_heads;
  a.block_size = block_size; a.bs_log2 = log2_exact(block_size);
  a.scale = scale;
  a.header = nullptr; a.items = nullptr; a.tok_split = nullptr; a.counters = nullptr;
  a.part_ml = nullptr; a.part_acc = nullptr;
  a.direct = 1;
  a.shared_items = nullptr;
  a.n_shared = 0;
  a.out_row_elems = static_cast<long long>(q_heads) * head_dim;
  a.out_col0 = 0;
  for (int p = 0; p < kMaxPeers; ++p) { a.peer_out[p] = nullptr; a.peer_flags[p] = nullptr; }
  a.n_peers = 0; a.my_rank = 0; a.epoch = 0;
  a.new_k = nullptr; a.new_v = nullptr; a.slots = nullptr;
  a.host_err = nullptr;
  a.pool_rows = 1ull << 30;
}

void attach_workspace(DecodeArgs& a, void* workspace, const WsLayout& w) {
  char* base = static_cast<char*>(workspace);
  a.header = reinterpret_cast<const PlanHeader*>(base);
  a.tok_split = reinterpret_cast<const TokSplit*>(base + w.off_tok);
  a.counters = reinterpret_cast<int*>(base + w.off_cnt);
  a.items = reinterpret_cast<const WorkItem*>(base + w.off_items);
  a.part_ml = reinterpret_cast<float*>(base + w.off_ml);
  a.part_acc = reinterpret_cast<float*>(base + w.off_acc);
  a.direct = 0;
}

int persistent_grid() {
  static thread_local int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms * 4;
}

// Budget of extra items for this workspace: what fits, capped by the target grid.
int plan_budget(int n_tokens, int q_heads, int kv_heads, int head_dim, size_t workspace_bytes, WsLayout* w) {
  const int fit = ws_extra_for_bytes(n_tokens, q_heads, kv_heads, head_dim, workspace_bytes, max_extra(kv_heads));
  if (fit < 0) return -1;
  *w = ws_layout(n_tokens, q_heads, kv_heads, head_dim, fit);
  const int target_extra = (tuning().target_ctas + kv_heads - 1) / kv_heads;
  return fit < target_extra ? fit : target_extra;
}

int plan_device(const int* token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim, void* workspace,
                size_t workspace_bytes, cudaStream_t stream, pkv_decode_plan* plan, const RouteArgs* route = nullptr) {
  if (!token_pos || !workspace || !plan) return fail(PKV_E_ARG, "pkv_decode_plan_device: null pointer");
  std::memset(plan, 0, sizeof(*plan));
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(PKV_E_ARG, "pkv_decode_plan_device: workspace must be 256-byte aligned");
  WsLayout w;
  const int budget = plan_budget(n_tokens, q_heads, kv_heads, head_dim, workspace_bytes, &w);
  if (budget < 0)
    return fail(PKV_E_WORKSPACE, "pkv_decode_plan_device: workspace of %zu bytes cannot hold the plan for %d tokens", workspace_bytes, n_tokens);
  char* base = static_cast<char*>(workspace);
  if (route)
    decode_plan_kernel<true><<<1, kPlanThreads, 0, stream>>>(
        token_pos, n_tokens, kv_heads, budget, tuning().wave_ctas, tuning().forced_chunk,
        reinterpret_cast<PlanHeader*>(base), reinterpret_cast<TokSplit*>(base + w.off_tok),
        reinterpret_cast<int*>(base + w.off_cnt), reinterpret_cast<WorkItem*>(base + w.off_items), *route);
  else
    decode_plan_kernel<false><<<1, kPlanThreads, 0, stream>>>(
        token_pos, n_tokens, kv_heads, budget, tuning().wave_ctas, tuning().forced_chunk,
        reinterpret_cast<PlanHeader*>(base), reinterpret_cast<TokSplit*>(base + w.off_tok),
        reinterpret_cast<int*>(base + w.off_cnt), reinterpret_cast<WorkItem*>(base + w.off_items), RouteArgs{});
  int st = check_launch("decode_plan_kernel");
  if (st != PKV_OK) return st;
  plan->n_tokens = n_tokens; plan->q_heads = q_heads; plan->kv_heads = kv_heads; plan->head_dim = head_dim;
  plan->chunk = -1;                      // decided on the device
  plan->n_items = n_tokens + budget;     // upper bound
  plan->exact = 0;
  plan->reserved = 1;                    // tokens may have been split: run the merge
  return PKV_OK;
}

struct FusedAppend {
  const void* k;
  const void* v;
  const int* slots;
};

struct PeerSetup {
  void* const* out;      // host array: every rank's full output buffer (device pointers valid on this GPU)
  int* const* flags;     // host array: every rank's flag array
  int n_peers, my_rank, epoch, q_heads_total;
};

template <typename T>
int decode_planned(const pkv_decode_plan* plan, const void* q, const void* kc, const void* vc, const int* bt,
                   const int* to, const int* ts, const int* tp, void* out, int block_size, float scale,
                   void* workspace, size_t workspace_bytes, pkv_stream stream, const PeerSetup* peers = nullptr,
                   const FusedAppend* app = nullptr, bool may_allocate = true) {
  const char* fn = peers ? "pkv_decode_attn_planned_peer" : (app ? "pkv_append_decode_attn_planned" : "pkv_decode_attn_planned");
  if (!plan) return fail(PKV_E_ARG, "%s: null plan", fn);
  if (plan->n_tokens <= 0) return PKV_OK;
  int st = check_error_mirror(fn);
  if (st != PKV_OK) return st;
  st = validate_geometry(fn, plan->n_tokens, plan->q_heads, plan->kv_heads, plan->head_dim, block_size);
  if (st != PKV_OK) return st;
  st = validate_pointers(fn, q, kc, vc, bt, to, ts, tp, out, sizeof(T) * static_cast<size_t>(plan->head_dim));
  if (st != PKV_OK) return st;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255)) return fail(PKV_E_ARG, "%s: workspace null or not 256-byte aligned", fn);
  WsLayout w;
  if (plan_budget(plan->n_tokens, plan->q_heads, plan->kv_heads, plan->head_dim, workspace_bytes, &w) < 0)
    return fail(PKV_E_WORKSPACE, "%s: workspace of %zu bytes is smaller than the plan it should hold", fn, workspace_bytes);
  DecodeArgs a;
  fill_args(a, q, kc, vc, bt, to, ts, tp, out, plan->n_tokens, plan->q_heads, plan->kv_heads, plan->head_dim, block_size, scale);
  attach_workspace(a, workspace, w);
  a.host_err = error_mirror(may_allocate);
  if (plan->num_blocks > 0) a.pool_rows = static_cast<unsigned long long>(plan->num_blocks) * block_size;
  if (peers) {
    if constexpr (sizeof(T) != 2) return fail(PKV_E_UNSUPPORTED, "%s: the head-sharded exchange is for 16-bit outputs", fn);
    if (peers->n_peers < 1 || peers->n_peers > kMaxPeers || peers->my_rank < 0 || peers->my_rank >= peers->n_peers)
      return fail(PKV_E_ARG, "%s: rank %d of %d (at most %d)", fn, peers->my_rank, peers->n_peers, kMaxPeers);
    if (peers->q_heads_total != plan->q_heads * peers->n_peers || (plan->head_dim & 3))
      return fail(PKV_E_ARG, "%s: %d heads in all must be %d ranks x %d local heads, head_dim a multiple of 4", fn,
                  peers->q_heads_total, peers->n_peers, plan->q_heads);
    for (int p = 0; p < peers->n_peers; ++p) {
      if (!peers->out[p] || !peers->flags[p]) return fail(PKV_E_ARG, "%s: null peer pointer for rank %d", fn, p);
      if ((reinterpret_cast<uintptr_t>(peers->out[p]) & 15) || (reinterpret_cast<uintptr_t>(peers->flags[p]) & 3))
        return fail(PKV_E_ARG, "%s: rank %d's output buffer must be 16-byte aligned and its flags 4-byte aligned", fn, p);
      a.peer_out[p] = peers->out[p];
      a.peer_flags[p] = peers->flags[p];
    }
    if (peers->out[peers->my_rank] != out) return fail(PKV_E_ARG, "%s: out must be this rank's own full buffer", fn);
    a.n_peers = peers->n_peers; a.my_rank = peers->my_rank; a.epoch = peers->epoch;
    a.out_row_elems = static_cast<long long>(peers->q_heads_total) * plan->head_dim;
    a.out_col0 = peers->my_rank * plan->q_heads * plan->head_dim;
  }
  if (app) {
    if (!app->k || !app->v || !app->slots) return fail(PKV_E_ARG, "%s: null k, v or slots", fn);
    if (!tma_path<T>(a))
      return fail(PKV_E_UNSUPPORTED, "%s: the fused append runs on the TMA kernel only (16-bit K/V, head_dim 64 or 128, at most 16 "
                  "query heads per kv head, power-of-two block_size >= 16); call pkv_append_* first instead", fn);
    if (!aligned16(app->k) || !aligned16(app->v)) return fail(PKV_E_ARG, "%s: k and v must be 16-byte aligned", fn);
    a.new_k = app->k; a.new_v = app->v; a.slots = app->slots;
  }
  const int n_shared = plan->reserved >> 1;
  if (n_shared > 0) {
    if (!shared_units_ok<T>(a))
      return fail(PKV_E_UNSUPPORTED, "%s: a plan with shared-prefix units needs 16-bit K/V, head_dim 64, at most 8 query heads per kv head "
                  "and a power-of-two block_size >= 16", fn);
    a.shared_items = reinterpret_cast<const int4*>(a.items + plan->n_items);
    a.n_shared = n_shared;
  }
  if (plan->cluster >= 2 && !peers && n_shared == 0 && a.head_dim == 64 && a.group <= 8 && tma_path<T>(a)) {
    bool launched = false;
    st = launch_tma_cluster<T>(a, plan->cluster, static_cast<cudaStream_t>(stream), &launched);
    if (st != PKV_OK || launched) return st;
  }
  long long blocks = static_cast<long long>(plan->n_items) * plan->kv_heads;
  if (!plan->exact && blocks > persistent_grid()) blocks = persistent_grid();
  if (blocks > 0x7fffffffll) blocks = 0x7fffffffll;
  return launch_decode<T>(a, static_cast<int>(blocks), static_cast<cudaStream_t>(stream), (plan->reserved & 1) != 0);
}

template <typename T>
int decode_all_in_one(const void* q, const void* kc, const void* vc, const int* bt, const int* to, const int* ts,
                      const int* tp, void* out, int n_tokens, int q_heads, int kv_heads, int head_dim,
                      int block_size, float scale, void* workspace, size_t workspace_bytes, pkv_stream stream,
                      bool may_allocate = true) {
  const char* fn = "pkv_decode_attn";
  if (n_tokens <= 0 || q_heads <= 0) return PKV_OK;  // the reference launchers' silent no-op
  int st = check_error_mirror(fn);
  if (st != PKV_OK) return st;
  st = validate_geometry(fn, n_tokens, q_heads, kv_heads, head_dim, block_size);
  if (st != PKV_OK) return st;
  st = validate_pointers(fn, q, kc, vc, bt, to, ts, tp, out, sizeof(T) * static_cast<size_t>(head_dim));
  if (st != PKV_OK) return st;
  if (!workspace) {
    DecodeArgs a;
    fill_args(a, q, kc, vc, bt, to, ts, tp, out, n_tokens, q_heads, kv_heads, head_dim, block_size, scale);
    a.host_err = error_mirror(may_allocate);
    long long blocks = static_cast<long long>(n_tokens) * kv_heads;
    if (blocks > 0x7fffffffll) blocks = 0x7fffffffll;
    return launch_decode<T>(a, static_cast<int>(blocks), static_cast<cudaStream_t>(stream), false);
  }
  pkv_decode_plan plan;
  st = plan_device(tp, n_tokens, q_heads, kv_heads, head_dim, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), &plan);
  if (st != PKV_OK) return st;
  return decode_planned<T>(&plan, q, kc, vc, bt, to, ts, tp, out, block_size, scale, workspace, workspace_bytes, stream,
                           nullptr, nullptr, may_allocate);
}

// ---- mixed steps ------------------------------------------------------------------------
int default_min_run() {
  static const int v = [] { const int e = env_int("PKV_MIXED_MIN_RUN", 16); return e < 1 ? 1 : e; }();
  return v;
}

// Router scratch behind the decode workspace: three int arrays of n_tokens, four of max_runs, the counts.
struct RouteLayout { size_t off_start, off_len, off_eff, off_qs, off_ql, off_ctx, off_tbl, off_dims, total; };
RouteLayout route_layout(int n_tokens) {
  RouteLayout r;
  const size_t arr = align256(sizeof(int) * static_cast<size_t>(n_tokens));
  r.off_start = 0; r.off_len = arr; r.off_eff = 2 * arr;
  r.off_qs = 3 * arr; r.off_ql = 4 * arr; r.off_ctx = 5 * arr; r.off_tbl = 6 * arr;
  r.off_dims = 7 * arr;
  r.total = 7 * arr + 256;
  return r;
}

template <typename T>
bool prefill_capable(int head_dim, int block_size, float scale) {
  if constexpr (IsF32<T>::value) return false;
  return head_dim == 64 && log2_exact(block_size) >= 4 && scale > 0.f && tensor_map_encoder() != nullptr;
}

template <typename T>
int mixed_attn(const void* q, const void* kc, const void* vc, const int* bt, const int* to, const int* ts, const int* tp,
               void* out, int n_tokens, int q_heads, int kv_heads, int head_dim, int block_size, int num_blocks,
               float scale, int min_run, void* workspace, size_t workspace_bytes, pkv_stream stream) {
  const char* fn = "pkv_mixed_attn";
  if (n_tokens <= 0 || q_heads <= 0) return PKV_OK;
  if (min_run <= 0) min_run = default_min_run();
  // Steps that cannot hold a prefill chunk, and geometries the prefill kernel does not run, are plain decode steps.
  if (n_tokens < min_run || !workspace || !prefill_capable<T>(head_dim, block_size, scale))
    return decode_all_in_one<T>(q, kc, vc, bt, to, ts, tp, out, n_tokens, q_heads, kv_heads, head_dim, block_size, scale,
                                workspace, workspace_bytes, stream);
  int st = check_error_mirror(fn);
  if (st != PKV_OK) return st;
  st = validate_geometry(fn, n_tokens, q_heads, kv_heads, head_dim, block_size);
  if (st != PKV_OK) return st;
  st = validate_pointers(fn, q, kc, vc, bt, to, ts, tp, out, sizeof(T) * static_cast<size_t>(head_dim));
  if (st != PKV_OK) return st;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(PKV_E_ARG, "%s: workspace must be 256-byte aligned", fn);
  const RouteLayout rl = route_layout(n_tokens);
  if (workspace_bytes < rl.total + ws_layout(n_tokens, q_heads, kv_heads, head_dim, 0).total)
    return fail(PKV_E_WORKSPACE, "%s: workspace of %zu bytes is too small for a step of %d tokens (pkv_mixed_attn_workspace_bytes)",
                fn, workspace_bytes, n_tokens);
  const size_t dec_bytes = (workspace_bytes - rl.total) & ~static_cast<size_t>(255);
  char* rbase = static_cast<char*>(workspace) + dec_bytes;
  RouteArgs r;
  r.token_seq = ts; r.table_offset = to;
  r.min_run = min_run; r.q_heads = q_heads;
  r.run_start = reinterpret_cast<int*>(rbase + rl.off_start);
  r.run_len = reinterpret_cast<int*>(rbase + rl.off_len);
  r.eff_len = reinterpret_cast<int*>(rbase + rl.off_eff);
  r.q_start = reinterpret_cast<int*>(rbase + rl.off_qs);
  r.q_len = reinterpret_cast<int*>(rbase + rl.off_ql);
  r.ctx_len = reinterpret_cast<int*>(rbase + rl.off_ctx);
  r.tbl_off = reinterpret_cast<int*>(rbase + rl.off_tbl);
  r.dims = reinterpret_cast<int*>(rbase + rl.off_dims);
  pkv_decode_plan plan;
  std::memset(&plan, 0, sizeof(plan));
  st = plan_device(tp, n_tokens, q_heads, kv_heads, head_dim, workspace, dec_bytes, static_cast<cudaStream_t>(stream), &plan, &r);
  if (st != PKV_OK) return st;
  plan.num_blocks = num_blocks > 0 ? num_blocks : 0;
  // decode tokens (and short runs) through the decode kernels; tokens of long runs are in no work item
  st = decode_planned<T>(&plan, q, kc, vc, bt, to, ts, tp, out, block_size, scale, workspace, dec_bytes, stream);
  if (st != PKV_OK) return st;
  // the long runs through the tensor-core kernel, whose item counts come from the router
  const int max_runs = n_tokens / min_run;
  if constexpr (!IsF32<T>::value)
    st = prefill_launch<T>(q, kc, vc, bt, r.tbl_off, r.q_start, r.q_len, r.ctx_len, out, n_tokens, max_runs, n_tokens,
                           q_heads, kv_heads, head_dim, block_size, num_blocks, scale, stream, r.dims, true);
  return st;
}

}  // namespace
}  // namespace pkv

using namespace pkv;

extern "C" {

int pkv_debug_device_flags(unsigned int* flags) {
  if (!flags) return fail(PKV_E_ARG, "pkv_debug_device_flags: null output");
  unsigned int v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_pkv_device_error, sizeof(v));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_pkv_device_error, &zero, sizeof(zero));
  if (e != cudaSuccess) return fail(PKV_E_CUDA, "pkv_debug_device_flags: %s", cudaGetErrorString(e));
  unsigned int pf = 0;
  const int st = pkv::prefill_read_flags(&pf);
  if (st != PKV_OK) return st;
  *flags = v | pf | pkv::take_error_mirror();
  return PKV_OK;
}

size_t pkv_decode_workspace_bytes(int n_tokens, int q_heads, int kv_heads, int head_dim) {
  if (n_tokens <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0) return 0;
  return ws_layout(n_tokens, q_heads, kv_heads, head_dim, max_extra(kv_heads)).total;
}

size_t pkv_decode_plan_staging_bytes(int n_tokens, int kv_heads) {
  if (n_tokens <= 0 || kv_heads <= 0) return 0;
  const WsLayout w = ws_layout(n_tokens, 1, kv_heads, 1, max_extra(kv_heads));
  return w.off_ml;  // header .. end of items
}

// Builds the plan image in host memory; *image_bytes is what has to reach the start of the workspace.
static int plan_host_image(const char* fn, const int* h_token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim,
                           void* h_staging, size_t staging_bytes, size_t workspace_bytes, pkv_decode_plan* plan,
                           size_t* image_bytes) {
  if (!plan) return fail(PKV_E_ARG, "%s: null plan", fn);
  std::memset(plan, 0, sizeof(*plan));
  *image_bytes = 0;
  if (n_tokens <= 0) return PKV_OK;
  if (!h_token_pos || !h_staging) return fail(PKV_E_ARG, "%s: null pointer", fn);
  int st = validate_geometry(fn, n_tokens, q_heads, kv_heads, head_dim, 1);
  if (st != PKV_OK) return st;
  WsLayout w;
  const int budget = plan_budget(n_tokens, q_heads, kv_heads, head_dim, workspace_bytes, &w);
  if (budget < 0) return fail(PKV_E_WORKSPACE, "%s: workspace of %zu bytes cannot hold the plan for %d tokens", fn, workspace_bytes, n_tokens);

  long long items_at[kNumChunkCandidates] = {0};
  for (int t = 0; t < n_tokens; ++t) {
    if (h_token_pos[t] < 0) return fail(PKV_E_ARG, "%s: token %d has negative position %d", fn, t, h_token_pos[t]);
    const int L = h_token_pos[t] + 1;
    for (int j = 0; j < kNumChunkCandidates; ++j) items_at[j] += (L + (kMinChunk << j) - 1) / (kMinChunk << j);
  }
  const int chunk = choose_chunk(items_at, n_tokens, kv_heads, budget, tuning().wave_ctas, tuning().forced_chunk);
  long long n_items = n_tokens;
  if (chunk > 0) {
    n_items = 0;
    for (int t = 0; t < n_tokens; ++t) n_items += (h_token_pos[t] + chunk) / chunk;
  }
  const size_t image = w.off_items + sizeof(WorkItem) * static_cast<size_t>(n_items);
  if (image > staging_bytes) return fail(PKV_E_WORKSPACE, "%s: staging buffer of %zu bytes is smaller than the %zu-byte plan image", fn, staging_bytes, image);

  char* img = static_cast<char*>(h_staging);
  std::memset(img, 0, w.off_items);
  PlanHeader* hd = reinterpret_cast<PlanHeader*>(img);
  TokSplit* tsp = reinterpret_cast<TokSplit*>(img + w.off_tok);
  WorkItem* it = reinterpret_cast<WorkItem*>(img + w.off_items);
  int ni = 0, np = 0;
  // Longest first: full-size chunks, then the ragged tails in decreasing length, so
  // that dealing the list round-robin gives every worker about the same number of
  // keys and the short units land at the end of the launch.  (Handing units out
  // dynamically through an atomic counter was measured and was no faster.)
  for (int t = 0; t < n_tokens; ++t) {
    const int L = h_token_pos[t] + 1;
    const int ns = chunk > 0 ? (L + chunk - 1) / chunk : 1;
    tsp[t] = TokSplit{np, ns};
    if (ns > 1) np += ns;
    if (chunk > 0)
      for (int s = 0; s + 1 < ns || (s < ns && L - s * chunk == chunk); ++s)
        it[ni++] = WorkItem{t, s * chunk, chunk, ns > 1 ? tsp[t].part_base + s : -1};
  }
  const int n_full = ni;
  for (int t = 0; t < n_tokens; ++t) {
    const int L = h_token_pos[t] + 1;
    const int ns = tsp[t].nsplits;
    const int b = chunk > 0 ? (ns - 1) * chunk : 0;
    const int len = L - b;
    if (chunk > 0 && len == chunk) continue;  // already listed as a full chunk
    it[ni++] = WorkItem{t, b, len, ns > 1 ? tsp[t].part_base + ns - 1 : -1};
  }
  std::stable_sort(it + n_full, it + ni, [](const WorkItem& x, const WorkItem& y) { return x.kv_len > y.kv_len; });
  hd->magic = kPlanMagic;
  hd->n_items = ni;
  hd->chunk = chunk;
  hd->n_tokens = n_tokens;
  hd->n_parts = np;
  hd->kv_heads = kv_heads;
  *image_bytes = image;
  plan->n_tokens = n_tokens; plan->q_heads = q_heads; plan->kv_heads = kv_heads; plan->head_dim = head_dim;
  plan->chunk = chunk;
  plan->n_items = ni;
  plan->exact = 1;
  plan->reserved = np > 0 ? 1 : 0;       // whether any token was split (the merge kernel is skipped otherwise)
  // Small steps: when every (token, kv head) can have a cluster of its own with all clusters resident at
  // once, and no warp of a cluster would get more than a few slabs, the attention call runs as clusters
  // and merges inside the launch (the image above stays valid: the call falls back to it if the device
  // turns the cluster launch down).
  if (cluster_form_enabled() && np > 0 && head_dim == 64 && q_heads / kv_heads <= 8) {
    const long long pairs = static_cast<long long>(n_tokens) * kv_heads;
    const long long resident = static_cast<long long>(persistent_sms()) * 3;
    if (pairs * 2 <= resident) {
      int cs = static_cast<int>(std::min<long long>(8, resident / pairs));
      if (tuning().cluster_size >= 2 && tuning().cluster_size < cs) cs = tuning().cluster_size;
      while (cs > 2 && !cluster_size_ok(cs)) --cs;       // 8, 4, 3 or 2 blocks: what the landing areas are sized for
      int max_len = 0;
      for (int t = 0; t < n_tokens; ++t) max_len = std::max(max_len, h_token_pos[t] + 1);
      if ((max_len + 4 * cs - 1) / (4 * cs) <= tuning().cluster_max_keys) plan->cluster = cs;
    }
  }
  return PKV_OK;
}

int pkv_decode_plan_host(const int* h_token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim,
                         void* h_staging, size_t staging_bytes, void* workspace, size_t workspace_bytes,
                         pkv_stream stream, pkv_decode_plan* plan) {
  const char* fn = "pkv_decode_plan_host";
  if (n_tokens > 0 && !workspace) return fail(PKV_E_ARG, "%s: null pointer", fn);
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(PKV_E_ARG, "%s: workspace must be 256-byte aligned", fn);
  size_t image = 0;
  const int st = plan_host_image(fn, h_token_pos, n_tokens, q_heads, kv_heads, head_dim, h_staging, staging_bytes,
                                 workspace_bytes, plan, &image);
  if (st != PKV_OK || image == 0) return st;
  const cudaError_t e = cudaMemcpyAsync(workspace, h_staging, image, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(PKV_E_CUDA, "%s: plan upload failed: %s", fn, cudaGetErrorString(e));
  return PKV_OK;
}

int pkv_decode_plan_host_image(const int* h_token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim,
                               void* h_staging, size_t staging_bytes, size_t workspace_bytes, pkv_decode_plan* plan,
                               size_t* image_bytes) {
  if (!image_bytes) return fail(PKV_E_ARG, "pkv_decode_plan_host_image: null image_bytes");
  return plan_host_image("pkv_decode_plan_host_image", h_token_pos, n_tokens, q_heads, kv_heads, head_dim, h_staging,
                         staging_bytes, workspace_bytes, plan, image_bytes);
}

int pkv_decode_plan_host_shared(const int* h_token_pos, const int* h_token_seq, const int* h_tables,
                                const int* h_table_offset, int n_tokens, int n_seqs, int n_table, int block_size,
                                int q_heads, int kv_heads, int head_dim, long long min_saved_bytes, void* h_staging,
                                size_t staging_bytes, void* workspace, size_t workspace_bytes, pkv_stream stream,
                                pkv_decode_plan* plan) {
  const char* fn = "pkv_decode_plan_host_shared";
  if (!plan) return fail(PKV_E_ARG, "%s: null plan", fn);
  std::memset(plan, 0, sizeof(*plan));
  if (n_tokens <= 0) return PKV_OK;
  if (!h_token_pos || !h_token_seq || !h_tables || !h_table_offset || !h_staging || !workspace)
    return fail(PKV_E_ARG, "%s: null pointer", fn);
  int st = validate_geometry(fn, n_tokens, q_heads, kv_heads, head_dim, block_size);
  if (st != PKV_OK) return st;
  if (n_seqs <= 0 || n_table < 0) return fail(PKV_E_ARG, "%s: n_seqs %d, n_table %d", fn, n_seqs, n_table);
  const int bsl = log2_exact(block_size);
  // Shared units run on the TMA kernel only; any other geometry gets the ordinary plan.
  if (head_dim != 64 || q_heads / kv_heads > 8 || bsl < 4)
    return pkv_decode_plan_host(h_token_pos, n_tokens, q_heads, kv_heads, head_dim, h_staging, staging_bytes, workspace,
                                workspace_bytes, stream, plan);
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(PKV_E_ARG, "%s: workspace must be 256-byte aligned", fn);
  WsLayout w;
  const int budget = plan_budget(n_tokens, q_heads, kv_heads, head_dim, workspace_bytes, &w);
  if (budget < 0) return fail(PKV_E_WORKSPACE, "%s: workspace of %zu bytes cannot hold the plan for %d tokens", fn, workspace_bytes, n_tokens);

  // ---- 1. which tokens share a prefix: sequences with the same first block form a cluster; what the
  //         cluster shares is the longest run of leading blocks common to all its members, cut below
  //         every member's own position (a token's newest key is never shared) ----
  constexpr int kMinShared = 64;                // keys; below this a shared unit is not worth its partial
  std::vector<int> seq_tokens(n_seqs, 0);
  for (int t = 0; t < n_tokens; ++t) {
    if (h_token_pos[t] < 0) return fail(PKV_E_ARG, "%s: token %d has negative position %d", fn, t, h_token_pos[t]);
    if (h_token_seq[t] < 0 || h_token_seq[t] >= n_seqs) return fail(PKV_E_ARG, "%s: token %d names sequence %d of %d", fn, t, h_token_seq[t], n_seqs);
    ++seq_tokens[h_token_seq[t]];
  }
  auto table_len = [&](int s) { return (s + 1 < n_seqs ? h_table_offset[s + 1] : n_table) - h_table_offset[s]; };
  std::vector<int> order;                       // decode tokens (one per sequence), sorted by first block
  for (int t = 0; t < n_tokens; ++t) {
    const int s = h_token_seq[t];
    if (seq_tokens[s] == 1 && table_len(s) > 0 && h_token_pos[t] >= kMinShared) order.push_back(t);
  }
  auto first_block = [&](int t) { return h_tables[h_table_offset[h_token_seq[t]]]; };
  std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return first_block(x) < first_block(y); });
  std::vector<int> shared_len(n_tokens, 0);     // keys of token t that a shared unit covers
  struct Group { int n_tok; int tok[kSharedTokens]; int len; };
  std::vector<Group> groups;
  for (size_t i = 0; i < order.size();) {
    size_t j = i + 1;
    while (j < order.size() && first_block(order[j]) == first_block(order[i])) ++j;
    if (j - i >= 2) {
      const int* t0 = h_tables + h_table_offset[h_token_seq[order[i]]];
      int lcp = table_len(h_token_seq[order[i]]), min_pos = h_token_pos[order[i]];
      for (size_t m = i + 1; m < j; ++m) {
        const int s = h_token_seq[order[m]];
        const int* tm = h_tables + h_table_offset[s];
        const int lim = std::min(lcp, table_len(s));
        int b = 0;
        while (b < lim && tm[b] == t0[b]) ++b;
        lcp = b;
        min_pos = std::min(min_pos, h_token_pos[order[m]]);
      }
      const long long keys = std::min<long long>(static_cast<long long>(lcp) << bsl, min_pos);
      const int len = static_cast<int>(keys) & ~15;
      if (len >= kMinShared) {
        size_t m = i;
        while (j - m >= 2) {                    // groups of four; a remainder of one stays an ordinary token
          Group g;
          g.n_tok = static_cast<int>(std::min<size_t>(kSharedTokens, j - m));
          if (j - m == kSharedTokens + 1) g.n_tok = 3;   // 5 = 3 + 2 rather than 4 + 1
          g.len = len;
          for (int k = 0; k < kSharedTokens; ++k) g.tok[k] = k < g.n_tok ? order[m + k] : order[m];
          for (int k = 0; k < g.n_tok; ++k) shared_len[order[m + k]] = len;
          groups.push_back(g);
          m += g.n_tok;
        }
      }
    }
    i = j;
  }
  // Shared units cost one more launch and a few more partials per token; they pay once the K/V reads
  // they save outweigh that (measured on B200: about 128 MiB per layer, where a 126 MB L2 already
  // serves most re-reads of a small shared prefix).
  long long saved = 0;
  for (const Group& g : groups) saved += static_cast<long long>(g.len) * (g.n_tok - 1) * kv_heads * head_dim * 2 * 2;
  if (min_saved_bytes < 0) min_saved_bytes = 128ll << 20;
  if (groups.empty() || saved < min_saved_bytes)
    return pkv_decode_plan_host(h_token_pos, n_tokens, q_heads, kv_heads, head_dim, h_staging, staging_bytes, workspace,
                                workspace_bytes, stream, plan);

  // ---- 2. chunk size: the ordinary rule over the ranges that are left, shared ranges counted once ----
  long long items_at[kNumChunkCandidates] = {0};
  auto count = [&](int len) {
    if (len > 0)
      for (int j = 0; j < kNumChunkCandidates; ++j) items_at[j] += (len + (kMinChunk << j) - 1) / (kMinChunk << j);
  };
  for (int t = 0; t < n_tokens; ++t) count(h_token_pos[t] + 1 - shared_len[t]);
  for (const Group& g : groups) count(g.len);
  int chunk = choose_chunk(items_at, n_tokens, kv_heads, budget, tuning().wave_ctas, tuning().forced_chunk);
  const int eff_chunk = chunk > 0 ? chunk : 0x40000000;
  auto nchunks = [&](int len) { return (len + eff_chunk - 1) / eff_chunk; };

  // ---- 3. partial slots per token: its shared chunks first, then its own ----
  char* img = static_cast<char*>(h_staging);
  if (w.off_items > staging_bytes) return fail(PKV_E_WORKSPACE, "%s: staging buffer of %zu bytes is too small", fn, staging_bytes);
  std::memset(img, 0, w.off_items);
  PlanHeader* hd = reinterpret_cast<PlanHeader*>(img);
  TokSplit* tsp = reinterpret_cast<TokSplit*>(img + w.off_tok);
  long long n_items = 0, n_shared = 0;
  int np = 0;
  for (int t = 0; t < n_tokens; ++t) {
    const int own = h_token_pos[t] + 1 - shared_len[t];
    const int ns = nchunks(shared_len[t]) + nchunks(own);
    tsp[t] = TokSplit{np, ns};
    if (ns > 1) np += ns;
    n_items += nchunks(own);
  }
  for (const Group& g : groups) n_shared += nchunks(g.len);
  const size_t image = w.off_items + sizeof(WorkItem) * static_cast<size_t>(n_items + 3 * n_shared);
  if (n_items + 3 * n_shared > w.cap_items || np > w.cap_parts || image > staging_bytes)   // no room: the ordinary plan
    return pkv_decode_plan_host(h_token_pos, n_tokens, q_heads, kv_heads, head_dim, h_staging, staging_bytes, workspace,
                                workspace_bytes, stream, plan);
  WorkItem* it = reinterpret_cast<WorkItem*>(img + w.off_items);
  int ni = 0;
  for (int t = 0; t < n_tokens; ++t) {          // full chunks first ...
    const int own = h_token_pos[t] + 1 - shared_len[t], nsc = nchunks(shared_len[t]), nx = nchunks(own);
    for (int s = 0; s < nx; ++s) {
      const int len = std::min(eff_chunk, own - s * eff_chunk);
      if (len == eff_chunk) it[ni++] = WorkItem{t, shared_len[t] + s * eff_chunk, len, tsp[t].nsplits > 1 ? tsp[t].part_base + nsc + s : -1};
    }
  }
  const int n_full = ni;
  for (int t = 0; t < n_tokens; ++t) {          // ... then the ragged tails, longest first
    const int own = h_token_pos[t] + 1 - shared_len[t], nsc = nchunks(shared_len[t]), nx = nchunks(own);
    if (nx == 0) continue;
    const int b = (nx - 1) * eff_chunk, len = own - b;
    if (len == eff_chunk) continue;
    it[ni++] = WorkItem{t, shared_len[t] + b, len, tsp[t].nsplits > 1 ? tsp[t].part_base + nsc + nx - 1 : -1};
  }
  std::stable_sort(it + n_full, it + ni, [](const WorkItem& x, const WorkItem& y) { return x.kv_len > y.kv_len; });
  SharedItem* sh = reinterpret_cast<SharedItem*>(it + ni);
  int nsh = 0;
  for (const Group& g : groups)
    for (int c = 0; c < nchunks(g.len); ++c) {
      SharedItem x;
      x.kv_begin = c * eff_chunk;
      x.kv_len = std::min(eff_chunk, g.len - c * eff_chunk);
      x.n_tok = g.n_tok;
      x.pad = 0;
      for (int k = 0; k < kSharedTokens; ++k) {
        x.token[k] = g.tok[k];
        x.part[k] = tsp[g.tok[k]].part_base + c;
      }
      sh[nsh++] = x;
    }
  hd->magic = kPlanMagic;
  hd->n_items = ni;
  hd->chunk = chunk;
  hd->n_tokens = n_tokens;
  hd->n_parts = np;
  hd->kv_heads = kv_heads;
  cudaError_t e = cudaMemcpyAsync(workspace, img, image, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(PKV_E_CUDA, "%s: plan upload failed: %s", fn, cudaGetErrorString(e));
  plan->n_tokens = n_tokens; plan->q_heads = q_heads; plan->kv_heads = kv_heads; plan->head_dim = head_dim;
  plan->chunk = chunk;
  plan->n_items = ni;
  plan->exact = 1;
  plan->reserved = (np > 0 ? 1 : 0) | (nsh << 1);   // bit 0: some token was split; the rest: shared units behind the items
  return PKV_OK;
}

int pkv_decode_plan_device(const int* token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim,
                           void* workspace, size_t workspace_bytes, pkv_stream stream, pkv_decode_plan* plan) {
  if (!plan) return fail(PKV_E_ARG, "pkv_decode_plan_device: null plan");
  std::memset(plan, 0, sizeof(*plan));
  if (n_tokens <= 0) return PKV_OK;
  int st = validate_geometry("pkv_decode_plan_device", n_tokens, q_heads, kv_heads, head_dim, 1);
  if (st != PKV_OK) return st;
  return plan_device(token_pos, n_tokens, q_heads, kv_heads, head_dim, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream), plan);
}

// Device address of g_builtin_scratch on the current device, looked up once per device.
static int builtin_scratch_address(void** out) {
  static std::mutex mu;
  static void* addr[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return fail(PKV_E_CUDA, "pkv_decode_attn_bf16_builtin_scratch: no current device");
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_builtin_scratch);
    if (e != cudaSuccess || !p)
      return fail(PKV_E_CUDA, "pkv_decode_attn_bf16_builtin_scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    addr[dev] = p;
  }
  *out = addr[dev];
  return PKV_OK;
}

int pkv_decode_attn_bf16_builtin_scratch(const void* q, const void* k_cache, const void* v_cache,
                                         const int* block_tables, const int* table_offset, const int* token_seq,
                                         const int* token_pos, void* out, int n_tokens, int q_heads, int kv_heads,
                                         int head_dim, int block_size, float scale, pkv_stream stream) {
  const char* fn = "pkv_decode_attn_bf16_builtin_scratch";
  if (n_tokens <= 0 || q_heads <= 0) return PKV_OK;
  int st = validate_geometry(fn, n_tokens, q_heads, kv_heads, head_dim, block_size);
  if (st != PKV_OK) return st;
  // The step's plan plus room for one GPU-wide wave of extra split-K items must fit.
  const int min_extra = (tuning().wave_ctas / 3 + kv_heads - 1) / kv_heads;
  const size_t need = ws_layout(n_tokens, q_heads, kv_heads, head_dim, min_extra).total;
  if (need > kBuiltinScratchBytes)
    return fail(PKV_E_WORKSPACE,
                "%s: a step of %d tokens x %d heads x head_dim %d needs %zu bytes of scratch, the built-in area holds %zu; "
                "use pkv_decode_attn_bf16 with a caller-owned workspace",
                fn, n_tokens, q_heads, head_dim, need, kBuiltinScratchBytes);
  void* ws = nullptr;
  st = builtin_scratch_address(&ws);
  if (st != PKV_OK) return st;
  // may_allocate = false: the pinned word that mirrors give-ups is used only if another call created it
  return decode_all_in_one<__nv_bfloat16>(q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out,
                                          n_tokens, q_heads, kv_heads, head_dim, block_size, scale, ws,
                                          kBuiltinScratchBytes, stream, false);
}

#define PKV_DECODE_ENTRY(SUFFIX, TYPE)                                                                               \
  int pkv_decode_attn_##SUFFIX(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,     \
                               const int* table_offset, const int* token_seq, const int* token_pos, void* out,      \
                               int n_tokens, int q_heads, int kv_heads, int head_dim, int block_size, float scale,  \
                               void* workspace, size_t workspace_bytes, pkv_stream stream) {                        \
    return decode_all_in_one<TYPE>(q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out,      \
                                   n_tokens, q_heads, kv_heads, head_dim, block_size, scale, workspace,             \
                                   workspace_bytes, stream);                                                        \
  }                                                                                                                  \
  int pkv_decode_attn_planned_##SUFFIX(const pkv_decode_plan* plan, const void* q, const void* k_cache,             \
                                       const void* v_cache, const int* block_tables, const int* table_offset,       \
                                       const int* token_seq, const int* token_pos, void* out, int block_size,       \
                                       float scale, void* workspace, size_t workspace_bytes, pkv_stream stream) {   \
    return decode_planned<TYPE>(plan, q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out,   \
                                block_size, scale, workspace, workspace_bytes, stream);                             \
  }

PKV_DECODE_ENTRY(f16, __half)
PKV_DECODE_ENTRY(bf16, __nv_bfloat16)
PKV_DECODE_ENTRY(f32, float)

#define PKV_DECODE_PEER_ENTRY(SUFFIX, TYPE)                                                                          \
  int pkv_decode_attn_planned_peer_##SUFFIX(const pkv_decode_plan* plan, const void* q, const void* k_cache,        \
                                            const void* v_cache, const int* block_tables, const int* table_offset,  \
                                            const int* token_seq, const int* token_pos, void* const* peer_out,      \
                                            int* const* peer_flags, int n_peers, int my_rank, int epoch,            \
                                            int q_heads_total, int block_size, float scale, void* workspace,        \
                                            size_t workspace_bytes, pkv_stream stream) {                            \
    if (!peer_out || !peer_flags || n_peers < 1 || my_rank < 0 || my_rank >= n_peers)                               \
      return fail(PKV_E_ARG, "pkv_decode_attn_planned_peer: null peer arrays or rank %d of %d", my_rank, n_peers);  \
    const PeerSetup ps{peer_out, peer_flags, n_peers, my_rank, epoch, q_heads_total};                               \
    return decode_planned<TYPE>(plan, q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos,        \
                                peer_out[my_rank], block_size, scale, workspace, workspace_bytes, stream, &ps);     \
  }

PKV_DECODE_PEER_ENTRY(f16, __half)
PKV_DECODE_PEER_ENTRY(bf16, __nv_bfloat16)

#define PKV_APPEND_DECODE_ENTRY(SUFFIX, TYPE)                                                                        \
  int pkv_append_decode_attn_planned_##SUFFIX(const pkv_decode_plan* plan, const void* q, const void* k,            \
                                              const void* v, const int* slots, void* k_cache, void* v_cache,        \
                                              const int* block_tables, const int* table_offset,                     \
                                              const int* token_seq, const int* token_pos, void* out,                \
                                              int block_size, float scale, void* workspace,                         \
                                              size_t workspace_bytes, pkv_stream stream) {                          \
    const FusedAppend app{k, v, slots};                                                                              \
    return decode_planned<TYPE>(plan, q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out,   \
                                block_size, scale, workspace, workspace_bytes, stream, nullptr, &app);              \
  }

PKV_APPEND_DECODE_ENTRY(f16, __half)
PKV_APPEND_DECODE_ENTRY(bf16, __nv_bfloat16)

unsigned long long pkv_debug_cluster_launches(void) { return pkv::g_cluster_launches.load(std::memory_order_relaxed); }

size_t pkv_mixed_attn_workspace_bytes(int n_tokens, int q_heads, int kv_heads, int head_dim) {
  if (n_tokens <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0) return 0;
  return pkv_decode_workspace_bytes(n_tokens, q_heads, kv_heads, head_dim) + route_layout(n_tokens).total;
}

#define PKV_MIXED_ENTRY(SUFFIX, TYPE)                                                                                \
  int pkv_mixed_attn_##SUFFIX(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,      \
                              const int* table_offset, const int* token_seq, const int* token_pos, void* out,       \
                              int n_tokens, int q_heads, int kv_heads, int head_dim, int block_size, int num_blocks, \
                              float scale, int min_run, void* workspace, size_t workspace_bytes, pkv_stream stream) { \
    return mixed_attn<TYPE>(q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out, n_tokens,    \
                            q_heads, kv_heads, head_dim, block_size, num_blocks, scale, min_run, workspace,          \
                            workspace_bytes, stream);                                                                \
  }

PKV_MIXED_ENTRY(f16, __half)
PKV_MIXED_ENTRY(bf16, __nv_bfloat16)

}  // extern "C"
