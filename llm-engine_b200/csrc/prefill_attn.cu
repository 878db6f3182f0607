// Paged (chunked) prefill attention entry points (include/pkv.h, section a3).
#include "launch_util.hpp"
#include "status.hpp"

extern "C" {
int pkv_prefill_attn_bf16(const void*, const void*, const void*, const int*, const int*, const int*, const int*,
                          const int*, void*, int, int, int, int, int, int, int, float, pkv_stream) {
  return pkv::fail(PKV_E_UNSUPPORTED, "pkv_prefill_attn_bf16: kernel not built into this library");
}
int pkv_prefill_attn_f16(const void*, const void*, const void*, const int*, const int*, const int*, const int*,
                         const int*, void*, int, int, int, int, int, int, int, float, pkv_stream) {
  return pkv::fail(PKV_E_UNSUPPORTED, "pkv_prefill_attn_f16: kernel not built into this library");
}
}
