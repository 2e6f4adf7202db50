// Helpers shared by the torch-facing host layer: dtype tags, stream fetch,
// C-ABI status -> exception. Nothing here launches work.
#pragma once

#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <cuda_runtime_api.h>

#include <cstdlib>
#include <cstring>
#include <optional>
#include <string>

#include "pla_b200.h"

namespace pla_ops {

inline int dtype_tag(const at::Tensor& t, const char* name) {
  switch (t.scalar_type()) {
    case at::kBFloat16: return PLA_B200_BF16;
    case at::kHalf: return PLA_B200_F16;
    case at::kFloat: return PLA_B200_F32;
    default: TORCH_CHECK(false, name, " must be bf16, fp16 or fp32, got ", t.scalar_type());
  }
}

inline void* stream_of(const at::Tensor& t) {
  return static_cast<void*>(c10::cuda::getCurrentCUDAStream(t.device().index()).stream());
}

inline void check_abi(int rc, const char* op) {
  TORCH_CHECK(rc == PLA_B200_OK, op, ": ", pla_b200_last_error());
}

// PLA_BYPASS_EXEC=1 (read once): every op validates its arguments and returns without launching, to
// measure a serving stack's host overhead (src/bypass_exec.h of the reference).
inline bool bypass_exec() {
  static const bool on = [] {
    const char* v = std::getenv("PLA_BYPASS_EXEC");
    return v != nullptr && std::strcmp(v, "1") == 0;   // exactly "1", as in the reference
  }();
  return on;
}

// PLA_SANITY_CHECK=1 (read at every call, as in the reference: src/sanity_check.h): value-level checks of
// the index metadata on the host. They synchronise the stream and copy to the host: a debugging aid.
// While the current stream is being captured into a CUDA graph the checks are skipped (a copy to the host would
// invalidate the capture), as the reference does; a failing capture-status query raises.
inline bool sanity_check() {
  const char* v = std::getenv("PLA_SANITY_CHECK");
  if (v == nullptr || std::strcmp(v, "1") != 0) return false;
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  const cudaError_t err = cudaStreamIsCapturing(c10::cuda::getCurrentCUDAStream().stream(), &capture);
  TORCH_CHECK(err == cudaSuccess, "PLA_SANITY_CHECK: cudaStreamIsCapturing failed: ", cudaGetErrorString(err));
  return capture == cudaStreamCaptureStatusNone;
}

// Value checks on host copies of the index metadata. They return a message (empty = fine) and the op raises
// it from its own frame.
// Offsets must start at 0, never decrease, and end within `tokens`; intervals longer than `t_max` (> 0) fail.
inline std::string sanity_offsets(const at::Tensor& cu, int64_t tokens, int64_t t_max) {
  const at::Tensor h = cu.to(at::kCPU).to(at::kLong).contiguous();
  const int64_t* p = h.data_ptr<int64_t>();
  const int64_t n = h.numel();
  if (n < 1 || p[0] != 0) return "offsets must start at 0";
  for (int64_t i = 1; i < n; ++i) {
    if (p[i] < p[i - 1]) return "offsets decrease at entry " + std::to_string(i);
    if (t_max > 0 && p[i] - p[i - 1] > t_max)
      return "interval " + std::to_string(i - 1) + " is longer than " + std::to_string(t_max);
  }
  if (p[n - 1] > tokens) return "offsets run past the " + std::to_string(tokens) + " token rows";
  return std::string();
}

// Slot indices must be below `slots` (negative values are padding).
inline std::string sanity_slots(const at::Tensor& idx, int64_t slots) {
  const at::Tensor h = idx.to(at::kCPU).to(at::kLong).contiguous();
  const int64_t* p = h.data_ptr<int64_t>();
  for (int64_t i = 0; i < h.numel(); ++i)
    if (p[i] >= slots)
      return "slot index " + std::to_string(p[i]) + " at entry " + std::to_string(i) + " is outside the pool of " +
             std::to_string(slots);
  return std::string();
}

inline void check_cuda(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}

inline void check_same_device(const at::Tensor& ref, const std::optional<at::Tensor>& t, const char* name) {
  if (t.has_value() && t->defined())
    TORCH_CHECK(t->device() == ref.device(), name, " must be on the same device as q");
}

inline const int32_t* i32_ptr(const std::optional<at::Tensor>& t, const char* name) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->scalar_type() == at::kInt, name, " must be int32");
  return t->data_ptr<int32_t>();
}

}  // namespace pla_ops
