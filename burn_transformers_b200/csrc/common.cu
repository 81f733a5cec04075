#include "common.cuh"
#include <atomic>
#include <cstdarg>
#include <cstdlib>

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
bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("BT_NO_PDL");
    return !(v && v[0] == '1');
  }();
  return on;
}
static std::atomic<long long> g_launches{0};
int sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (counts[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) counts[dev] = n;
  }
  return counts[dev];
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }
}  // namespace bt

extern "C" long long bt_launch_count() { return bt::launches(); }
extern "C" const char* bt_last_error() { return bt::error_buffer(); }

// Compile-time facts a caller can check after loading the library.
extern "C" int bt_abi_version() { return 1; }
