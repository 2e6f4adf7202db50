// Shared device helpers for the sm_100a kernels: mbarrier + bulk-copy (TMA
// engine) wrappers with bounded waits, dtype loaders, gate and norm math.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/pla_b200.h"

namespace pla {

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);

#define PLA_REQUIRE(cond, code, ...)   \
  do {                                 \
    if (!(cond)) {                     \
      ::pla::set_error(__VA_ARGS__);   \
      return (code);                   \
    }                                  \
  } while (0)

#define PLA_CUDA_OK(expr)                                                        \
  do {                                                                           \
    cudaError_t err__ = (expr);                                                  \
    if (err__ != cudaSuccess) {                                                  \
      ::pla::set_error("%s failed: %s", #expr, cudaGetErrorString(err__));       \
      return PLA_B200_E_CUDA;                                                    \
    }                                                                            \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int sm_count();  // multiprocessors of the current device (cached per device)
// Device address of the library's own status word on the current GPU (NULL when it cannot be resolved):
// every entry point substitutes it for a NULL `status` argument.
int32_t* device_status_word();
template <typename Args>
inline void default_status(Args& a) {
  if (a.status == nullptr) a.status = device_status_word();
}

// -------------------------------------------------------------- device side
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}

// Makes mbarrier initialisation visible to the async (bulk-copy) proxy.
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// "Done once per device" flags for a kernel's launch attributes (dynamic shared memory size), shared by the host
// threads that may call an entry point at the same time. Devices past the table are configured on every call.
struct DeviceOnce {
  std::atomic<bool> done[64];
  bool needed(int dev) const { return dev < 0 || dev >= 64 || !done[dev].load(std::memory_order_acquire); }
  void mark(int dev) {
    if (dev >= 0 && dev < 64) done[dev].store(true, std::memory_order_release);
  }
};

// Asks for the 128-byte line at `p` to be brought into L2 (no register, no dependency: a hint that lets the DRAM
// fetch of data needed a phase later run under the current phase).
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Bounded wait: gives up after `limit` polls (each poll itself blocks for a
// hardware-defined slice), returning false so the caller can flag a timeout
// instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// 1-D bulk copy global -> shared, completion counted on `bar`. Addresses and
// size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_addr(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}

// 1-D bulk copy shared -> global (bulk async-group completion).
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_addr(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's bulk groups still READ shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Orders generic-proxy shared-memory writes before later async-proxy reads.
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- dtypes
template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) {
  return __bfloat162float(x);
}
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) {
  return __half2float(x);
}
template <>
__device__ __forceinline__ float to_f32<float>(float x) {
  return x;
}

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) {
  return __float2half_rn(x);
}
template <>
__device__ __forceinline__ float from_f32<float>(float x) {
  return x;
}

// Load element `i` of an array whose dtype is only known at run time.
__device__ __forceinline__ float load_any(const void* p, int dtype, int64_t i) {
  if (dtype == PLA_B200_F32) return static_cast<const float*>(p)[i];
  if (dtype == PLA_B200_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

// 4 consecutive 16-bit activations -> float4 (8-byte load; caller guarantees alignment).
template <typename T>
__device__ __forceinline__ float4 load4(const T* p) {
  uint2 raw = *reinterpret_cast<const uint2*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
  return make_float4(to_f32(e[0]), to_f32(e[1]), to_f32(e[2]), to_f32(e[3]));
}

// ---------------------------------------------------------------- math
// 2^x on the special-function unit, flushing denormals: a single instruction. (`__expf` is this after a multiply by
// log2 e, but without the flush it expands to a handful of instructions around the same unit.)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_exp(float x) { return fast_exp2(x * 1.4426950408889634f); }
__device__ __forceinline__ float sigmoidf_fast(float x) { return __fdividef(1.0f, 1.0f + fast_exp(-x)); }

// log-decay g (<= 0): the state is multiplied by exp(g).
//   softplus form: g = -exp(A_log) * softplus(x), softplus with (beta, threshold)
//   safe form:     g = lower_bound * sigmoid(exp(A_log) * x)
// x = a + dt_bias. (src/pla_device_helpers.cuh:215-246)
__device__ __forceinline__ float log_decay(float x, float A_log, int gate, float sp_beta,
                                           float sp_thr, float lower_bound) {
  const float eA = fast_exp(A_log);
  if (gate == PLA_B200_GATE_SAFE) {
    // exp(A_log)*x formed as 0 when x == 0 so that a huge A_log cannot give inf*0
    // (src/decode/kda_replayssm/kda_mtp_verify.cu:88-92).
    const float z = (x == 0.0f) ? 0.0f : eA * x;
    return lower_bound * sigmoidf_fast(z);
  }
  const float bx = sp_beta * x;
  const float sp = (bx <= sp_thr) ? (1.0f / sp_beta) * __logf(1.0f + fast_exp(bx)) : x;
  return -eA * sp;
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

__device__ __forceinline__ float dot4(const float4& a, const float4& b) {
  return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
}

}  // namespace pla
