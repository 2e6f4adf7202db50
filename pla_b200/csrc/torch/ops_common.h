// Helpers shared by the torch-facing host layer: dtype tags, stream fetch,
// C-ABI status -> exception. Nothing here launches work.
#pragma once

#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <optional>

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
