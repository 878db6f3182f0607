// Host-visible record of bounded waits that ran out.
//
// Every wait inside the kernels is bounded; a wait that runs out leaves a bit in a device word
// (pkv_debug_device_flags reads it, synchronising) and, so that the caller learns of it without
// synchronising, in one pinned host word that the kernels can store to.  The attention entry points
// look at that word before they enqueue anything: the call that follows an incomplete launch
// returns PKV_E_CUDA once (the word is cleared by the report), in the manner of CUDA's own
// asynchronous errors.  The launch after that runs normally: nothing is disabled.
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "status.hpp"

namespace pkv {
namespace {
std::mutex g_mu;
unsigned int* g_mirror = nullptr;   // cudaHostAlloc'd (portable, mapped): one word, valid on every device
bool g_tried = false;
unsigned int g_plain = 0;           // what pkv_debug_set_reported_flags recorded (works without a device)
}  // namespace

// The pinned word, created on first use when `create` is set.  The one allocating call this makes
// (cudaHostAlloc of 64 bytes, once per process) is kept away from callers that must not allocate:
// they pass create = false and get the word only if somebody else made it already.
unsigned int* error_mirror(bool create) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_mirror || !create || g_tried) return g_mirror;
  g_tried = true;
  void* p = nullptr;
  if (cudaHostAlloc(&p, 64, cudaHostAllocPortable | cudaHostAllocMapped) == cudaSuccess && p) {
    std::memset(p, 0, 64);
    __atomic_store_n(&g_mirror, static_cast<unsigned int*>(p), __ATOMIC_RELEASE);
  } else {
    cudaGetLastError();
  }
  return g_mirror;
}

unsigned int take_error_mirror() {
  // the common case -- nothing recorded -- is two plain loads, no lock and no write
  unsigned int* m = __atomic_load_n(&g_mirror, __ATOMIC_ACQUIRE);
  if (__atomic_load_n(&g_plain, __ATOMIC_RELAXED) == 0 && (!m || __atomic_load_n(m, __ATOMIC_RELAXED) == 0)) return 0;
  std::lock_guard<std::mutex> lock(g_mu);
  unsigned int v = g_plain;
  g_plain = 0;
  if (g_mirror) v |= __atomic_exchange_n(g_mirror, 0u, __ATOMIC_ACQ_REL);
  return v;
}

int check_error_mirror(const char* fn) {
  const unsigned int v = take_error_mirror();
  if (!v) return PKV_OK;
  return fail(PKV_E_CUDA,
              "%s: an earlier launch gave up on a bounded wait (flags 0x%x: 1 TMA producer, 2 tile consumer, 4 prefill "
              "pipeline, 8 peer GPU) and left its output incomplete; this call enqueued nothing, the next one runs normally",
              fn, v);
}

}  // namespace pkv

extern "C" int pkv_debug_set_reported_flags(unsigned int flags) {
  std::lock_guard<std::mutex> lock(pkv::g_mu);
  pkv::g_plain |= flags;
  return PKV_OK;
}
