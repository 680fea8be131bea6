// Library-wide pieces of the C ABI: version, error text, cached device facts.
#include <cstring>

#include "bt_common.cuh"

namespace bt {

namespace {
thread_local char g_err[512] = {0};
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices] = {0};
}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

namespace {
int g_dependent_launch = 1;
}
int dependent_launch_mode() { return g_dependent_launch; }

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

}  // namespace bt

extern "C" int bt_version(void) { return 100; }  // 0.1.0

extern "C" const char* bt_last_error(void) { return bt::g_err; }

extern "C" int bt_sm_count(void) { return bt::sm_count(); }

extern "C" int bt_set_dependent_launch(int enable) {
  const int prev = bt::g_dependent_launch;
  if (enable >= 0) bt::g_dependent_launch = enable ? 1 : 0;
  return prev;
}
