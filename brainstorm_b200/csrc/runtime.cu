// Error reporting and device queries shared by every entry point of the C ABI.
#include "common.cuh"

#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace brt_b200 {

char* error_buffer() {
  static thread_local char buf[1024] = {0};
  return buf;
}

static std::atomic<uint64_t> g_launches{0};

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

uint64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

// ---- optional per-kernel timing ----------------------------------------------------------
namespace {
struct TimedLaunch {
  const char* name;
  cudaEvent_t start, stop;
};
std::atomic<int> g_profiling{0};
std::mutex g_profile_mutex;
std::vector<TimedLaunch*> g_timed;
}  // namespace

KernelTimer::KernelTimer(const char* name, cudaStream_t stream) : stream_(stream), slot_(nullptr) {
  if (!g_profiling.load(std::memory_order_relaxed)) return;
  TimedLaunch* t = new TimedLaunch{name, nullptr, nullptr};
  if (cudaEventCreate(&t->start) != cudaSuccess || cudaEventCreate(&t->stop) != cudaSuccess ||
      cudaEventRecord(t->start, stream) != cudaSuccess) {
    if (t->start) cudaEventDestroy(t->start);
    if (t->stop) cudaEventDestroy(t->stop);
    delete t;
    cudaGetLastError();
    return;
  }
  slot_ = t;
}

KernelTimer::~KernelTimer() {
  if (slot_ == nullptr) return;
  TimedLaunch* t = static_cast<TimedLaunch*>(slot_);
  cudaEventRecord(t->stop, stream_);
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  g_timed.push_back(t);
}

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

BRT_API int brt_abi_version(void) { return 3; }

BRT_API const char* brt_last_error(void) { return brt_b200::error_buffer(); }

BRT_API uint64_t brt_kernel_launch_count(void) { return brt_b200::launch_count(); }

BRT_API void brt_profile_enable(int on) { brt_b200::g_profiling.store(on ? 1 : 0); }

BRT_API int brt_profile_report(char* out, size_t out_bytes) {
  using namespace brt_b200;
  clear_error();
  BRT_REQUIRE(out != nullptr && out_bytes > 2, "no room for the report");
  std::vector<TimedLaunch*> taken;
  {
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    taken.swap(g_timed);
  }
  std::map<std::string, std::pair<long, double>> sums;  // name -> (launches, total ms)
  for (TimedLaunch* t : taken) {
    float ms = 0.f;
    if (cudaEventSynchronize(t->stop) == cudaSuccess &&
        cudaEventElapsedTime(&ms, t->start, t->stop) == cudaSuccess) {
      auto& s = sums[t->name];
      s.first += 1;
      s.second += ms;
    }
    cudaEventDestroy(t->start);
    cudaEventDestroy(t->stop);
    delete t;
  }
  std::string text = "{";
  for (const auto& kv : sums) {
    char item[256];
    snprintf(item, sizeof(item), "%s\"%s\": {\"launches\": %ld, \"total_ms\": %.6f}",
             text.size() > 1 ? ", " : "", kv.first.c_str(), kv.second.first, kv.second.second);
    text += item;
  }
  text += "}";
  BRT_REQUIRE(text.size() + 1 <= out_bytes, "report needs %zu bytes", text.size() + 1);
  memcpy(out, text.c_str(), text.size() + 1);
  return BRT_OK;
}

}  // extern "C"
