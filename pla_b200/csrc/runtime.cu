// Library-wide host helpers: thread-local error text, device property cache.
#include <stdarg.h>

#include <atomic>
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
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return 148;
  if (dev < 64 && cached[dev].load(std::memory_order_relaxed) != 0) return cached[dev].load(std::memory_order_relaxed);
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  if (dev < 64) cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

// Library-owned status word: kernels OR their PLA_B200_DEV_* bits into it when the caller passed no status
// pointer, so that a timeout or a bad slot is never silent. One per GPU, sticky until cleared.
__device__ int32_t g_device_status;

int32_t* device_status_word() {
  static std::atomic<int32_t*> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return nullptr;
  if (dev < 64) {
    int32_t* hit = cached[dev].load(std::memory_order_acquire);
    if (hit != nullptr) return hit;
  }
  void* addr = nullptr;
  if (cudaGetSymbolAddress(&addr, g_device_status) != cudaSuccess) return nullptr;
  if (dev < 64) cached[dev].store(static_cast<int32_t*>(addr), std::memory_order_release);
  return static_cast<int32_t*>(addr);
}

}  // namespace pla

extern "C" int pla_b200_device_status(int32_t* out, int clear) {
  using namespace pla;
  PLA_REQUIRE(out != nullptr, PLA_B200_E_INVALID, "out is NULL");
  int32_t* word = device_status_word();
  PLA_REQUIRE(word != nullptr, PLA_B200_E_CUDA, "the status word's address is not available on this device");
  PLA_CUDA_OK(cudaMemcpy(out, word, sizeof(int32_t), cudaMemcpyDeviceToHost));   // synchronises with prior work
  if (clear) PLA_CUDA_OK(cudaMemset(word, 0, sizeof(int32_t)));
  return PLA_B200_OK;
}

extern "C" const char* pla_b200_last_error(void) { return pla::g_error; }
extern "C" int pla_b200_abi_version(void) { return PLA_B200_ABI_VERSION; }
