/*
 * pkv.h -- C ABI of the B200 (sm_100a) paged-KV hot path for llm-engine.
 *
 * This is the whole drop-in boundary: plain pointers and sizes, no C++ or
 * framework types.  Every entry point returns a status code (0 = PKV_OK,
 * negative = error, see pkv_status_string / pkv_last_error), never throws,
 * never synchronises the device (pkv_debug_device_flags excepted) and enqueues
 * its work on the CUDA stream it is given (NULL = the legacy default stream,
 * which is what llm-engine passes at every call site,
 * src/model/cuda/cuda_model.cu:347-390).  Device memory is allocated in two
 * places only, both set-up code outside the per-step calls: pkv_peer_alloc /
 * pkv_peer_open (buffers of the head-sharded exchange) and the grow-only scratch
 * behind the three engine::launch_* symbols the library also exports for an
 * unmodified llm-engine (their signatures carry no workspace argument).  All data
 * pointers are DEVICE pointers unless a parameter is named h_* or documented as
 * host memory.
 *
 * Each declaration names the llm-engine interface it replaces (file:line within
 * that project).  Layout conventions are llm-engine's own:
 *   - K and V pools are separate arrays [num_blocks*block_size slots][kv_heads][head_dim],
 *     row-major (src/model/cuda/cuda_model.cu:276-285, src/model/cpu/cpu_model.cpp:83-87);
 *   - slot(pos) = block_table[pos / block_size] * block_size + pos % block_size
 *     (include/engine/kv_cache.h:29-31);
 *   - q / out rows are [n_tokens][q_heads][head_dim]; query head h reads kv head
 *     h / (q_heads / kv_heads) (include/engine/ops.h:79-86);
 *   - block_tables is the step's concatenation of every distinct sequence's
 *     table, table_offset[s] its start, token_seq[t] the step-local sequence of
 *     packed token t, token_pos[t] its absolute position; a token attends
 *     positions 0..token_pos[t] inclusive (include/engine/cuda_kernels.h:44-53).
 */
#ifndef PKV_H_
#define PKV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PKV_ABI_VERSION 2

typedef void* pkv_stream; /* a cudaStream_t */

enum pkv_status {
  PKV_OK = 0,
  PKV_E_ARG = -1,         /* null pointer, negative size, misaligned pointer */
  PKV_E_UNSUPPORTED = -2, /* geometry outside what the kernels implement */
  PKV_E_WORKSPACE = -3,   /* workspace missing or too small for the request */
  PKV_E_CUDA = -4,        /* the CUDA runtime refused the launch or a copy */
  PKV_E_NOMEM = -5,       /* block pool exhausted (host bookkeeping) */
  PKV_E_STATE = -6        /* handle used in a way its state does not allow */
};

int pkv_abi_version(void);
/* Static description of a status code. */
const char* pkv_status_string(int status);
/* Detail of the calling thread's most recent failure ("" if none). */
const char* pkv_last_error(void);

/* Bounded waits.  Every wait inside the kernels has a limit; a wait that runs out
 * makes its warp or block wind down (tensor memory released, no trap) and leaves the
 * launch's output incomplete.  The record of it is a bit -- 1: a TMA producer never saw
 * its ring slot released; 2: a consumer never saw its tile arrive; 4: a prefill
 * pipeline wait; 8: a peer GPU's flag in the head-sharded exchange -- kept in two
 * places: a device word, and one pinned host word the kernels store to.  The attention
 * entry points (pkv_decode_attn_*, the planned, fused, peer and mixed forms,
 * pkv_prefill_attn_*) look at the host word before they enqueue anything: the first
 * such call after an incomplete launch has reached the host returns PKV_E_CUDA once,
 * with the bits in pkv_last_error(), and enqueues nothing; the record is cleared by
 * that report and the next call runs normally (nothing is disabled).  The three
 * engine::launch_* symbols turn it into their std::runtime_error.
 *
 * pkv_debug_device_flags is the one entry point that SYNCHRONISES the device: it
 * reads and clears both records (0: no kernel gave up).
 * pkv_debug_set_reported_flags is a testing aid: it makes the next attention call
 * behave as if a kernel had recorded `flags` (works without a GPU).
 * No llm-engine counterparts. */
int pkv_debug_device_flags(unsigned int* flags);
int pkv_debug_set_reported_flags(unsigned int flags);
/* How many attention launches of this process took the cluster form (pkv_decode_plan.cluster): a
 * plan that asks for it on a device that cannot hold all the clusters at once silently takes the
 * ordinary form, and this counter is how a test tells the two apart.  No llm-engine counterpart. */
unsigned long long pkv_debug_cluster_launches(void);

/* ----------------------------------------------------------- K/V append ----
 * K/V append.  Replaces engine::launch_store_kv (include/engine/cuda_kernels.h:43-45,
 * src/kernels/store_kv.cu:20-36) and the CPU memcpy pair
 * (src/model/cpu/cpu_model.cpp:153-157):
 *     k_cache[slots[t]][:] = k[t][:],  v_cache[slots[t]][:] = v[t][:]   for t < n_tokens.
 * Bit-exact byte copy; duplicate slots are allowed only with identical payloads
 * (llm-engine re-writes a shared full block with the same values,
 * src/scheduler/scheduler.cpp:60).  n_tokens <= 0 or kv_dim <= 0 is a no-op
 * returning PKV_OK, as in the reference launcher. */
int pkv_append_f16(const void* k, const void* v, const int* slots, void* k_cache, void* v_cache,
                   int n_tokens, int kv_dim, pkv_stream stream);
int pkv_append_bf16(const void* k, const void* v, const int* slots, void* k_cache, void* v_cache,
                    int n_tokens, int kv_dim, pkv_stream stream);
int pkv_append_f32(const void* k, const void* v, const int* slots, void* k_cache, void* v_cache,
                   int n_tokens, int kv_dim, pkv_stream stream);

/* -------------------------------------------------------- RoPE + append ----
 * RoPE fused into the append.  Replaces the three launches llm-engine makes per layer,
 * launch_rope(q), launch_rope(k), launch_store_kv (src/model/cuda/cuda_model.cu:366-368,
 * src/kernels/rope.cu:32-62; arithmetic of ref::rope_inplace, include/engine/ops.h:56-68):
 *   q[t][h][:]  <- rope(q[t][h][:], positions[t])            for the q_heads heads, in place
 *   k_cache[slots[t]][h][:] <- rope(k[t][h][:], positions[t]) for the kv_heads heads
 *   v_cache[slots[t]][:]    <- v[t][:]
 * with x'[i] = x[i]*cos - x[i+D/2]*sin, x'[i+D/2] = x[i+D/2]*cos + x[i]*sin (rotate_half
 * pairing), cos/sin = fp32 tables [max_positions][D/2] as built by ref::RopeTables
 * (include/engine/ops.h:34-51).  Products are rounded separately (no fused multiply-add),
 * so fp32 results equal the CPU code's bit for bit and 16-bit results equal its fp32 result
 * rounded once.  Unlike the reference, `k` itself is left unrotated (nothing reads it
 * after the append, src/model/cuda/cuda_model.cu:368-377).  head_dim must be even. */
int pkv_rope_append_f16(void* q, const void* k, const void* v, const int* positions, const float* cos_table,
                        const float* sin_table, const int* slots, void* k_cache, void* v_cache, int n_tokens,
                        int q_heads, int kv_heads, int head_dim, pkv_stream stream);
int pkv_rope_append_bf16(void* q, const void* k, const void* v, const int* positions, const float* cos_table,
                         const float* sin_table, const int* slots, void* k_cache, void* v_cache, int n_tokens,
                         int q_heads, int kv_heads, int head_dim, pkv_stream stream);
int pkv_rope_append_f32(void* q, const void* k, const void* v, const int* positions, const float* cos_table,
                        const float* sin_table, const int* slots, void* k_cache, void* v_cache, int n_tokens,
                        int q_heads, int kv_heads, int head_dim, pkv_stream stream);

/* ----------------------------------------------------- decode attention ----
 * Paged decode attention.  Replaces engine::launch_attention_decode and
 * engine::launch_attention_decode_gqa (include/engine/cuda_kernels.h:48-62,
 * src/kernels/attention_decode.cu:133-161, src/kernels/attention_decode_gqa.cu:200-232);
 * the arithmetic it must agree with is ref::paged_attention_head
 * (include/engine/ops.h:87-111).  Arguments up to `stream` are the reference
 * launcher's; `workspace` is caller-owned scratch for split-K over long contexts:
 *   - workspace == NULL: every (token, kv head) is handled by one thread block
 *     over its whole history (correct for any length, slow for long ones);
 *   - otherwise at least pkv_decode_workspace_bytes(...) bytes, 256-byte aligned.
 *     It carries no state between calls of this all-in-one form.
 * n_tokens <= 0 is a no-op.  Geometry limits: q_heads % kv_heads == 0,
 * head_dim <= 256, block_size >= 1. */
size_t pkv_decode_workspace_bytes(int n_tokens, int q_heads, int kv_heads, int head_dim);

int pkv_decode_attn_f16(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                        const int* table_offset, const int* token_seq, const int* token_pos, void* out,
                        int n_tokens, int q_heads, int kv_heads, int head_dim, int block_size,
                        float scale, void* workspace, size_t workspace_bytes, pkv_stream stream);
int pkv_decode_attn_bf16(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                         const int* table_offset, const int* token_seq, const int* token_pos, void* out,
                         int n_tokens, int q_heads, int kv_heads, int head_dim, int block_size,
                         float scale, void* workspace, size_t workspace_bytes, pkv_stream stream);
int pkv_decode_attn_f32(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                        const int* table_offset, const int* token_seq, const int* token_pos, void* out,
                        int n_tokens, int q_heads, int kv_heads, int head_dim, int block_size,
                        float scale, void* workspace, size_t workspace_bytes, pkv_stream stream);

/* The same operation for callers that cannot hand over a workspace because they cannot
 * allocate one: code that runs where device allocation is off the table -- a serving
 * engine that gave every free byte of HBM to its block pool at start-up (a later
 * cudaMalloc fails or fragments), or a per-token loop where cudaMalloc's implicit
 * device synchronisation is not acceptable.  Split-K scratch is a fixed 32 MiB area
 * inside the library's device image (each GPU that loads the library holds it until
 * the process exits); this call allocates nothing and calls no allocating routine.
 * Limits and rules:
 *   - a step whose plan does not fit the area returns PKV_E_WORKSPACE with the sizes
 *     in pkv_last_error() (at head_dim 64: about 1,900 extra split items at 32 query
 *     heads, 4,400 at 14); use pkv_decode_attn_bf16 with your own workspace then;
 *   - the first call on each device looks the area's address up
 *     (cudaGetSymbolAddress, with that device current): make that first call before
 *     any stream capture begins.  The address is then kept per device ordinal for the
 *     life of the process, which is the life of the device's primary context: a
 *     process that calls cudaDeviceReset must not use this entry point afterwards;
 *   - every call on a device shares the one area and rebuilds all of it that it reads
 *     (the plan is rewritten at each call), so nothing needs clearing between calls,
 *     but two calls that overlap on the GPU (different streams) race: serialise them.
 * This entry point has no counterpart in llm-engine. */
int pkv_decode_attn_bf16_builtin_scratch(const void* q, const void* k_cache, const void* v_cache,
                                         const int* block_tables, const int* table_offset,
                                         const int* token_seq, const int* token_pos, void* out,
                                         int n_tokens, int q_heads, int kv_heads, int head_dim,
                                         int block_size, float scale, pkv_stream stream);

/* Plan-once form.  A decode step calls attention once per layer with the SAME
 * index arrays (src/model/cuda/cuda_model.cu:349-377), so the split-K work list
 * can be built once per step and reused by every layer.
 *
 * pkv_decode_plan_host builds the list on the host from the host copy of
 * token_pos that the caller already has before uploading it
 * (src/model/cuda/cuda_model.cu:434-447,479), writes its image to `h_staging`
 * (host memory, pinned for a truly asynchronous copy; at least
 * pkv_decode_plan_staging_bytes(n_tokens, kv_heads) bytes; must stay untouched
 * until the copy has run) and enqueues one host-to-device copy into `workspace`.
 * pkv_decode_plan_device does the same from the device copy of token_pos with a
 * single small kernel, for callers that hold no host copy.
 * The plan is valid for any number of pkv_decode_attn_planned_* calls on the
 * same stream with the same n_tokens / heads / head_dim / token_pos contents. */
typedef struct pkv_decode_plan {
  int n_tokens;
  int q_heads, kv_heads, head_dim;
  int chunk;      /* keys per work item; 0 = no splitting */
  int n_items;    /* exact item count when host-built, upper bound when device-built */
  int exact;      /* 1 if n_items is exact */
  int reserved;   /* internal: bit 0 set when some token was split; the other bits count shared-prefix units */
  int num_blocks; /* blocks in each K/V pool, or 0 if unknown.  The planners leave 0; a caller that sets it
                     before pkv_decode_attn_planned_* gets tensor maps bounded by the pool, so that a wrong
                     block id reads zeros instead of memory beyond it (llm-engine's launcher signature
                     carries no pool size, which is why this is optional) */
  int cluster;    /* blocks per thread-block cluster (2..8) for the small-step form of the attention launch: one
                     cluster per (token, kv head), the history cut into one range per warp of the cluster, the
                     split-K merge done inside the launch through the cluster's shared memory -- one launch per
                     layer and no workspace traffic.  0 = the ordinary form (split-K units + merge launch).
                     pkv_decode_plan_host[_image] sets it (to 2, 3, 4 or 8) when the step qualifies -- head_dim 64,
                     at most 8 query heads per kv head, every cluster resident at once, at most 256 keys per
                     warp -- unless the environment has PKV_DECODE_CLUSTER=0 (read at every call); the other
                     planners leave 0.  A caller may clear it; a launch the kernel or the device cannot take
                     (fp32 K/V, block_size < 16, clusters that would not all be resident) runs the ordinary form.
                     A captured launch of this form stays correct when replayed over later steps of the same
                     token count: it reads no plan, only token_pos.
                     No counterpart in llm-engine. */
  int pad[2];
} pkv_decode_plan;

size_t pkv_decode_plan_staging_bytes(int n_tokens, int kv_heads);
int pkv_decode_plan_host(const int* h_token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim,
                         void* h_staging, size_t staging_bytes, void* workspace, size_t workspace_bytes,
                         pkv_stream stream, pkv_decode_plan* plan);
int pkv_decode_plan_device(const int* token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim,
                           void* workspace, size_t workspace_bytes, pkv_stream stream,
                           pkv_decode_plan* plan);
/* pkv_decode_plan_host without the copy, for a caller that replays a captured CUDA graph:
 * the image is written to h_staging and *image_bytes says how much of it must be at the
 * start of the workspace before the attention calls run; the caller's own graph carries
 * that copy (a memcpy node from h_staging of any size >= *image_bytes, e.g. the whole
 * staging buffer).  workspace_bytes is the size of the workspace the plan is for. */
int pkv_decode_plan_host_image(const int* h_token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim,
                               void* h_staging, size_t staging_bytes, size_t workspace_bytes,
                               pkv_decode_plan* plan, size_t* image_bytes);
/* Append fused into the attention: pkv_append_* followed by pkv_decode_attn_planned_*
 * in ONE kernel chain less (the two calls of src/model/cuda/cuda_model.cu:368-377
 * folded together).  The work unit that reaches a token's newest key takes that
 * key's K/V row from k / v instead of the pool and writes it to pool row
 * slots[token]; the pools end up byte-identical to what pkv_append_* writes.  For
 * decode steps only: every sequence brings exactly one token (a sequence that
 * brings several needs its earlier new keys in the pool first: append, then
 * pkv_decode_attn_planned_*).  Runs where the TMA kernel runs (16-bit K/V, head_dim
 * 64 or 128, at most 16 query heads per kv head, block_size a power of two >= 16);
 * PKV_E_UNSUPPORTED otherwise, with nothing enqueued.
 * Ordering: the launch is a programmatic dependent of the kernel before it on the stream and
 * starts fetching the pools' rows of positions BELOW token_pos while that kernel is still
 * running; q, k, v and slots are read, and everything is written, only after it has completed.
 * So the rows of earlier positions must not be produced by the kernel directly before this call
 * -- they never are in a decode step: they were written by earlier steps, and a step starts with
 * uploads or planning that complete before anything behind them begins (and this library's
 * block copy does not release its dependents early, so a copy-on-write copy directly before
 * this call is safe).  A caller whose own kernel writes such rows directly before this call
 * and releases its dependents early (griddepcontrol.launch_dependents) puts any other
 * operation in between, or sets PKV_PDL=0. */
int pkv_append_decode_attn_planned_f16(const pkv_decode_plan* plan, const void* q, const void* k, const void* v,
                                       const int* slots, void* k_cache, void* v_cache, const int* block_tables,
                                       const int* table_offset, const int* token_seq, const int* token_pos,
                                       void* out, int block_size, float scale, void* workspace,
                                       size_t workspace_bytes, pkv_stream stream);
int pkv_append_decode_attn_planned_bf16(const pkv_decode_plan* plan, const void* q, const void* k, const void* v,
                                        const int* slots, void* k_cache, void* v_cache, const int* block_tables,
                                        const int* table_offset, const int* token_seq, const int* token_pos,
                                        void* out, int block_size, float scale, void* workspace,
                                        size_t workspace_bytes, pkv_stream stream);

/* Shared-prefix-aware plan.  llm-engine's prefix cache makes sequences with a
 * common prompt share their leading blocks (KVCacheManager::allocate_prompt,
 * src/kv_cache/block_allocator.cpp:28-78), yet its decode kernels fetch those
 * blocks once per sequence.  Given the host copies of the step's index arrays (the
 * outputs of pkv_step_pack: token_seq, the concatenated tables, table_offset),
 * this planner finds the decode tokens whose sequences start with the same blocks
 * and covers that range with units that fetch K/V once for up to four tokens; each
 * token's own remaining range is planned as usual and the partials are merged by
 * the same kernel.  The plan is consumed by pkv_decode_attn_planned_* exactly like
 * one from pkv_decode_plan_host; results agree with it to rounding (the same
 * keys, grouped differently).  Geometries the shared units do not cover (head_dim
 * other than 64, more than 8 query heads per kv head, block_size not a power of
 * two >= 16, fp32 K/V) and steps without shared prefixes get the ordinary plan, and
 * so do steps whose shared units would save fewer than min_saved_bytes of K/V reads
 * per layer (-1: the library's default, 128 MiB, below which the extra launch costs
 * more than the reads it saves on a B200; 0: always use them). */
int pkv_decode_plan_host_shared(const int* h_token_pos, const int* h_token_seq, const int* h_tables,
                                const int* h_table_offset, int n_tokens, int n_seqs, int n_table,
                                int block_size, int q_heads, int kv_heads, int head_dim,
                                long long min_saved_bytes, void* h_staging, size_t staging_bytes,
                                void* workspace, size_t workspace_bytes, pkv_stream stream,
                                pkv_decode_plan* plan);
int pkv_decode_attn_planned_f16(const pkv_decode_plan* plan, const void* q, const void* k_cache,
                                const void* v_cache, const int* block_tables, const int* table_offset,
                                const int* token_seq, const int* token_pos, void* out, int block_size,
                                float scale, void* workspace, size_t workspace_bytes, pkv_stream stream);
int pkv_decode_attn_planned_bf16(const pkv_decode_plan* plan, const void* q, const void* k_cache,
                                 const void* v_cache, const int* block_tables, const int* table_offset,
                                 const int* token_seq, const int* token_pos, void* out, int block_size,
                                 float scale, void* workspace, size_t workspace_bytes, pkv_stream stream);
int pkv_decode_attn_planned_f32(const pkv_decode_plan* plan, const void* q, const void* k_cache,
                                const void* v_cache, const int* block_tables, const int* table_offset,
                                const int* token_seq, const int* token_pos, void* out, int block_size,
                                float scale, void* workspace, size_t workspace_bytes, pkv_stream stream);

/* Mixed steps: prefill chunks and decode tokens in ONE call, as llm-engine's forward
 * pass makes it (src/model/cuda/cuda_model.cu:362-377: every packed token of the step
 * goes through launch_attention_decode; include/engine/sequence.h:74-89: prefill slices
 * first, then decode tokens; a slice's tokens are packed consecutively,
 * src/model/cuda/cuda_model.cu:434-447).  Arguments are those of pkv_decode_attn_* plus
 * the pool size (num_blocks, 0 if unknown) and min_run.  On the device, with no host
 * synchronisation, the planner finds the runs -- maximal stretches of packed tokens of
 * one sequence at consecutive positions; runs of at least min_run tokens (<= 0: the
 * library's default, 16) go to the tensor-core prefill kernel as (first row, length,
 * cached context) records, all other tokens to the decode kernels, and both write the
 * same `out`.  K/V of every token must already be in the pools (pkv_append_* first).
 * Results agree with pkv_decode_attn_* on the same step within the dtype's tolerance.
 * Steps shorter than min_run, a null workspace, and geometries the prefill kernel does
 * not run (head_dim other than 64, block_size not a power of two >= 16) take the
 * pkv_decode_attn_* path unchanged.  The workspace holds the split-K scratch and the
 * router's arrays: at least pkv_mixed_attn_workspace_bytes(...), 256-byte aligned.
 * engine::launch_attention_decode[_gqa] as exported by this library call this. */
size_t pkv_mixed_attn_workspace_bytes(int n_tokens, int q_heads, int kv_heads, int head_dim);
int pkv_mixed_attn_f16(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                       const int* table_offset, const int* token_seq, const int* token_pos, void* out,
                       int n_tokens, int q_heads, int kv_heads, int head_dim, int block_size, int num_blocks,
                       float scale, int min_run, void* workspace, size_t workspace_bytes, pkv_stream stream);
int pkv_mixed_attn_bf16(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                        const int* table_offset, const int* token_seq, const int* token_pos, void* out,
                        int n_tokens, int q_heads, int kv_heads, int head_dim, int block_size, int num_blocks,
                        float scale, int min_run, void* workspace, size_t workspace_bytes, pkv_stream stream);

/* -------------------------------------------------- head-sharded decode ----
 * Head-sharded decode over the GPUs of one box (one process per GPU).  The path
 * scales by sequence without any exchange, and that is what the benchmark reports;
 * this variant is for a configuration whose kv heads divide the GPU count and
 * whose caller shards heads (tensor parallelism): rank r holds the pools of kv
 * heads [r*kv_heads, (r+1)*kv_heads) only, computes q_heads local query heads for
 * ALL tokens, and every rank needs the full [n_tokens][q_heads_total*head_dim]
 * output.  No llm-engine counterpart (single GPU, src/model/cuda/cuda_model.cu:239).
 *
 * pkv_decode_attn_planned_peer_* is pkv_decode_attn_planned_* with the exchange
 * fused into its merge kernel: each finished output row is stored straight into
 * every rank's full buffer over NVLink (plain peer stores, 8 bytes each), then the
 * rank raises flag `my_rank` on every peer and waits, with a bound, until its own
 * n_peers flags show `epoch`; when the call's kernels have completed on the stream
 * the whole output is in peer_out[my_rank].  peer_out / peer_flags are HOST arrays
 * of n_peers device pointers as seen from this GPU (own buffer at index my_rank;
 * flags are n_peers + 1 ints per rank, zero-initialised); epoch must grow by one
 * per call, the same on every rank, or be 0: the calls are then counted on the
 * device (in the extra int), which lets a captured CUDA graph be replayed;
 * plan->q_heads is the local head count.  A rank may enter its next call while a
 * peer still reads the output of this one, so a caller whose consumer is not already
 * ordered before the peers' next call (tensor-parallel layers are, by the all-reduce
 * that follows the output projection) alternates two buffers.  A wait
 * that runs out sets bit 3 of pkv_debug_device_flags and the kernel returns.
 *
 * pkv_peer_alloc / open / close / free are the set-up helpers for such buffers
 * (cudaMalloc + CUDA IPC): the only entry points of the library that allocate or
 * map device memory; call them before the serving loop. */
int pkv_decode_attn_planned_peer_f16(const pkv_decode_plan* plan, const void* q, const void* k_cache,
                                     const void* v_cache, const int* block_tables, const int* table_offset,
                                     const int* token_seq, const int* token_pos, void* const* peer_out,
                                     int* const* peer_flags, int n_peers, int my_rank, int epoch,
                                     int q_heads_total, int block_size, float scale, void* workspace,
                                     size_t workspace_bytes, pkv_stream stream);
int pkv_decode_attn_planned_peer_bf16(const pkv_decode_plan* plan, const void* q, const void* k_cache,
                                      const void* v_cache, const int* block_tables, const int* table_offset,
                                      const int* token_seq, const int* token_pos, void* const* peer_out,
                                      int* const* peer_flags, int n_peers, int my_rank, int epoch,
                                      int q_heads_total, int block_size, float scale, void* workspace,
                                      size_t workspace_bytes, pkv_stream stream);
int pkv_peer_alloc(size_t bytes, void** ptr, void* handle64);
int pkv_peer_open(const void* handle64, void** ptr);
int pkv_peer_close(void* ptr);
int pkv_peer_free(void* ptr);

/* ---------------------------------------------------- prefill attention ----
 * Paged (chunked) prefill attention on the tensor cores.  llm-engine has no such
 * kernel (src/kernels/attention_prefill.cu:1 is a stub; prefill tokens go through
 * the decode launcher, src/model/cuda/cuda_model.cu:370-377); the result it must
 * agree with is still ref::paged_attention_head applied to every (token, head)
 * of the chunk (include/engine/ops.h:87-111).
 * Sequence s (step-local index, table at block_tables + table_offset[s]) brings
 * q_len[s] new tokens, packed as rows q_start[s] .. q_start[s]+q_len[s]-1 of q/out,
 * at absolute positions ctx_len[s] .. ctx_len[s]+q_len[s]-1; row i attends
 * positions 0 .. ctx_len[s]+i (causal over cached plus new tokens).  K/V of the
 * chunk must already be in the pool (pkv_append_* first, as the reference orders
 * store_kv before attention, src/model/cuda/cuda_model.cu:362-368).
 * n_tokens is the total number of packed rows of q / out, num_blocks the pool size
 * (both bound the TMA descriptors); max_q_len >= max_s q_len[s] sizes the grid (the
 * caller's chunk size, include/engine/scheduler.h:26).  bf16 and f16, head_dim 64,
 * block_size a power of two >= 16, q_heads % kv_heads == 0; other geometries return
 * PKV_E_UNSUPPORTED (such steps go through pkv_decode_attn_*, as in the reference).
 * The kernel is persistent.  Eager launches hand their work out through a ticket
 * counter that belongs to (device, stream): calls on one stream never share it in
 * time, calls on different streams never share it at all, so any number may overlap.
 * A call made during stream capture, or on the 65th distinct stream of a device,
 * deals its work in a fixed order instead and touches no shared counter, so a
 * captured graph may be replayed next to anything. */
int pkv_prefill_attn_bf16(const void* q, const void* k_cache, const void* v_cache,
                          const int* block_tables, const int* table_offset, const int* q_start,
                          const int* q_len, const int* ctx_len, void* out, int n_tokens, int n_seqs,
                          int max_q_len, int q_heads, int kv_heads, int head_dim, int block_size,
                          int num_blocks, float scale, pkv_stream stream);
int pkv_prefill_attn_f16(const void* q, const void* k_cache, const void* v_cache,
                         const int* block_tables, const int* table_offset, const int* q_start,
                         const int* q_len, const int* ctx_len, void* out, int n_tokens, int n_seqs,
                         int max_q_len, int q_heads, int kv_heads, int head_dim, int block_size,
                         int num_blocks, float scale, pkv_stream stream);

/* ----------------------------------------------------------- block copy ----
 * Prefix-cache copy-on-write block copy.  No llm-engine counterpart (it shares
 * full blocks only and therefore never copies, docs/design.md:36); semantics are
 * memcpy's: for each pair i, block src_dst_pairs[2i] is copied over block
 * src_dst_pairs[2i+1] in both pools.  Destinations must be distinct from each
 * other and from every source of the same call.  Bit-exact.
 * pkv_copy_blocks_layers does the same for n_caches pools at once (every layer's
 * K and V): d_cache_ptrs is a device array of n_caches pool base pointers. */
int pkv_copy_blocks_f16(void* k_cache, void* v_cache, const int* src_dst_pairs, int n_pairs,
                        int block_size, int kv_dim, pkv_stream stream);
int pkv_copy_blocks_bf16(void* k_cache, void* v_cache, const int* src_dst_pairs, int n_pairs,
                         int block_size, int kv_dim, pkv_stream stream);
int pkv_copy_blocks_f32(void* k_cache, void* v_cache, const int* src_dst_pairs, int n_pairs,
                        int block_size, int kv_dim, pkv_stream stream);
int pkv_copy_blocks_layers(void* const* d_cache_ptrs, int n_caches, const int* src_dst_pairs,
                           int n_pairs, size_t block_bytes, pkv_stream stream);

/* -------------------------------------------------- step indices (host) ----
 * Step-index packing (host).  Replaces the loop of CudaModel::upload_step_indices
 * (src/model/cuda/cuda_model.cu:453-473): sequences are numbered in order of
 * first appearance among the packed tokens, each distinct sequence's block table
 * is appended once to `tables`, and slots[i] = slot(tok_pos[i]).  All pointers
 * are HOST pointers.  tok_seq_key[i] identifies token i's sequence (the reference
 * compares Sequence pointers); tok_blocks[i] / tok_num_blocks[i] is that
 * sequence's block table.  Outputs: slots[n_tokens], token_seq[n_tokens],
 * tables[tables_cap], table_offset[offsets_cap]; *n_seqs and *n_table receive the
 * counts.  PKV_E_WORKSPACE if a capacity is too small; PKV_E_ARG if a position
 * lies beyond its table. */
int pkv_step_pack(int n_tokens, const uint64_t* tok_seq_key, const int32_t* const* tok_blocks,
                  const int* tok_num_blocks, const int* tok_pos, int block_size, int* slots,
                  int* token_seq, int* tables, size_t tables_cap, int* table_offset,
                  size_t offsets_cap, int* n_seqs, int* n_table);

/* ------------------------------------------------ step indices (device) ----
 * Step-index build on the device.  Replaces all of CudaModel::upload_step_indices
 * (src/model/cuda/cuda_model.cu:453-491): its O(N*S) host loop and its six
 * synchronous host-to-device copies per step, which is what stands between the
 * caller and a CUDA-graph decode step.  Every sequence's block table lives in one
 * row of a device-resident store d_seq_tables[max_rows][table_stride] with its
 * length in d_seq_nblocks[max_rows] (zero-initialised by the caller).  Per step the
 * host sends two small arrays of int32 triples (one copy, if it packs them in one
 * buffer):
 *   d_updates[n_updates][3] = { row, block_index, block_id }: that entry of the row
 *       is set and the row's length raised to block_index + 1; block_index = -1
 *       releases the row (length 0).  Releases are applied before sets.
 *   d_slices[n_slices][3]   = { row, first_position, length }: the step's packed
 *       tokens, slice after slice (a decode token is a slice of length 1).
 * Outputs, identical to what pkv_step_pack writes for the same tokens: positions,
 * token_seq, slots [sum of lengths], tables (each distinct row's table once, in order
 * of first appearance), table_offset [distinct rows]; d_counts[4] = { n_tokens,
 * n_seqs, n_table, status }, status = 0 or a bit set: 1 tables_cap too small,
 * 2 tokens_cap too small (nothing is written in those two cases), 4 a position
 * beyond its row's table (its slot is written as 0), 8 a row or block index out of
 * range (ignored).  One launch, nothing synchronises; at most 4096 slices. */
int pkv_step_pack_device(const int32_t* d_updates, int n_updates, const int32_t* d_slices, int n_slices,
                         int32_t* d_seq_tables, int32_t* d_seq_nblocks, int max_rows, int table_stride,
                         int block_size, int32_t* d_slots, int32_t* d_token_seq, int32_t* d_positions,
                         int tokens_cap, int32_t* d_tables, int tables_cap, int32_t* d_table_offset,
                         int32_t* d_counts, pkv_stream stream);

/* ---------------------------------------------------- block bookkeeping ----
 * KV block bookkeeping (host).  C handles over the C++ KVCacheManager / BlockTable
 * of include/pkv_kv_cache.hpp, which keep the public surface of llm-engine's
 * classes (include/engine/kv_cache.h:21-99, src/kv_cache/block_allocator.cpp:8-142)
 * and hand out identical block ids, hashes and statistics. */
typedef struct pkv_kvmgr pkv_kvmgr;
typedef struct pkv_table pkv_table;

pkv_kvmgr* pkv_kvmgr_create(int num_blocks, int block_size, int enable_prefix_caching); /* NULL on bad args */
void pkv_kvmgr_destroy(pkv_kvmgr* m);
pkv_table* pkv_table_create(void);
void pkv_table_destroy(pkv_table* t);

/* kv_cache.h:62 -- cached token count, or -1 when the pool cannot fit the prompt. */
int pkv_kvmgr_allocate_prompt(pkv_kvmgr* m, pkv_table* t, const int32_t* tokens, int n_tokens);
/* kv_cache.h:66 -- 1 on success, 0 when out of blocks. */
int pkv_kvmgr_ensure_slot(pkv_kvmgr* m, pkv_table* t, int num_tokens);
/* kv_cache.h:72 */
void pkv_kvmgr_commit_computed(pkv_kvmgr* m, pkv_table* t, const int32_t* tokens, int n_tokens, int num_computed);
/* kv_cache.h:76 */
void pkv_kvmgr_free(pkv_kvmgr* m, pkv_table* t);
/* kv_cache.h:79 */
int pkv_kvmgr_lookup_cached_prefix(const pkv_kvmgr* m, const int32_t* tokens, int n_tokens);
/* kv_cache.h:81, block_allocator.cpp:16-23 */
uint64_t pkv_hash_block(uint64_t prev_hash, const int32_t* tokens, int n);
/* kv_cache.h:46-55 */
int pkv_kvmgr_block_size(const pkv_kvmgr* m);
int pkv_kvmgr_num_total_blocks(const pkv_kvmgr* m);
int pkv_kvmgr_capacity_tokens(const pkv_kvmgr* m);
int pkv_kvmgr_num_free_blocks(const pkv_kvmgr* m);
int pkv_kvmgr_num_cached_blocks(const pkv_kvmgr* m);
int pkv_kvmgr_num_available_blocks(const pkv_kvmgr* m);
int pkv_kvmgr_num_used_blocks(const pkv_kvmgr* m);
/* kv_cache.h:34-40 -- out[5] = prefix_queries, prefix_hit_blocks, prefix_total_blocks,
 * evictions, allocation_failures */
void pkv_kvmgr_stats(const pkv_kvmgr* m, uint64_t out[5]);
int pkv_kvmgr_ref_count(const pkv_kvmgr* m, int block);

/* kv_cache.h:21-32 */
int pkv_table_num_blocks(const pkv_table* t);
int pkv_table_num_committed(const pkv_table* t);
const int32_t* pkv_table_blocks(const pkv_table* t);  /* valid until the table is next modified */
const uint64_t* pkv_table_hashes(const pkv_table* t);
int64_t pkv_table_slot(const pkv_table* t, int pos, int block_size);

/* Copy-on-write bookkeeping; additive, no llm-engine counterpart.
 * fork: `child` (empty) comes to share every block of `parent`, the partial last
 * block included (reference counts +1).
 * cow: call before writing position `write_pos` of `t`.  If that block is still
 * shared and not yet committed, `t` moves to a private block: returns 1 with
 * *src / *dst for pkv_copy_blocks_*, 0 when no copy is needed, PKV_E_NOMEM when
 * the pool is exhausted. */
int pkv_kvmgr_fork(pkv_kvmgr* m, const pkv_table* parent, pkv_table* child);
int pkv_kvmgr_cow(pkv_kvmgr* m, pkv_table* t, int write_pos, int* src, int* dst);

#ifdef __cplusplus
}
#endif
#endif /* PKV_H_ */
