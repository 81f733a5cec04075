#include "common.cuh"
#include <cstdarg>

namespace bt {
char* error_buffer() {
  static thread_local char buffer[512] = {0};
  return buffer;
}
int fail(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(error_buffer(), 512, fmt, args);
  va_end(args);
  return 1;
}
}  // namespace bt

extern "C" const char* bt_last_error() { return bt::error_buffer(); }

// Compile-time facts a caller can check after loading the library.
extern "C" int bt_abi_version() { return 1; }
