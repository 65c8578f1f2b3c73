// Error reporting and version entry points of the C ABI.
#include "common.cuh"

namespace sage {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace sage

extern "C" int sage_b200_version(void) { return SAGE_B200_VERSION; }

extern "C" const char* sage_b200_last_error(void) { return sage::error_buffer(); }
