// Error reporting and device queries shared by every entry point of the C ABI.
#include "common.cuh"

#include <atomic>
#include <cstring>

namespace brt_b200 {

char* error_buffer() {
  static thread_local char buf[1024] = {0};
  return buf;
}

static std::atomic<uint64_t> g_launches{0};

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

uint64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

void clear_error() { error_buffer()[0] = '\0'; }

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 1024, fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static thread_local int cached_dev = -1;
  static thread_local int cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

}  // namespace brt_b200

extern "C" {

BRT_API int brt_abi_version(void) { return 2; }

BRT_API const char* brt_last_error(void) { return brt_b200::error_buffer(); }

BRT_API uint64_t brt_kernel_launch_count(void) { return brt_b200::launch_count(); }

}  // extern "C"
