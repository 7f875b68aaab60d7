#include "common.h"

namespace gbh {
char* error_buf() {
  static thread_local char buf[1024] = {0};
  return buf;
}
}  // namespace gbh

GBH_API const char* gbh_last_error() { return gbh::error_buf(); }
