// Library-wide host helpers: thread-local error text, device property cache.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace pla {

namespace {
thread_local char g_error[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace pla

extern "C" const char* pla_b200_last_error(void) { return pla::g_error; }
extern "C" int pla_b200_abi_version(void) { return PLA_B200_ABI_VERSION; }
