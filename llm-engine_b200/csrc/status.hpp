// Status codes and the per-thread error message shared by every C-ABI entry point.
#pragma once
#include <cstdarg>
#include <cstdio>

#include "pkv.h"

namespace pkv {

// Records a printf-style message for pkv_last_error() and returns `code`.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();

}  // namespace pkv
