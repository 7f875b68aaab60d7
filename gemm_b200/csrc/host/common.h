// Shared declarations of the host-side library (libgb_host.so): C ABI export macro and the
// per-thread error string returned by gbh_last_error().
#pragma once
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string>

#define GBH_API extern "C" __attribute__((visibility("default")))

namespace gbh {
char* error_buf();
inline int fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buf(), 1024, fmt, ap);
  va_end(ap);
  return -1;
}
}  // namespace gbh
