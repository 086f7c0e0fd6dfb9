#include "common/rs_common.h"

namespace rs {
char* last_error_buf() {
  static thread_local char buf[1024] = {0};
  return buf;
}
int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 1024, fmt, ap);
  va_end(ap);
  return code;
}
}  // namespace rs

RS_API const char* rs_last_error() { return rs::last_error_buf(); }
RS_API int rs_abi_version() { return 1; }
