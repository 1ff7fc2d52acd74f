// Error reporting and device queries of the lightop_b200 C-ABI library.
#include "common.h"
#include <cstring>

namespace lo {

static thread_local char g_err[512] = "";
std::atomic<long long> g_launch_count{0};

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

}  // namespace lo

extern "C" int lo_version(void) { return 1; }
extern "C" const char *lo_last_error(void) { return lo::g_err; }
extern "C" int lo_sm_count(void) { return lo::sm_count(); }
extern "C" long long lo_launch_count(void) { return lo::g_launch_count.load(std::memory_order_relaxed); }
