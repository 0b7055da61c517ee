// Helpers shared by the *_binding.cpp files: argument checks that raise a
// Python RuntimeError (as the reference's TORCH_CHECK lines do,
// agent_workdir/kernels/axpby_binding.cpp:18-24) and translation of a launcher's
// int status into the same kind of error. Light torch headers only, as in the
// reference binding (agent_workdir/kernels/axpby_binding.cpp:1-5).
#pragma once

#include <torch/types.h>
#include <torch/csrc/utils/pybind.h>
#include <cuda_runtime.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGuard.h>

#include "../binding_registry.h"
#include "../../../include/cuda_agent_b200.h"

namespace cab_binding {

inline void check_cuda_contig(const torch::Tensor& t, const char* name, c10::ScalarType dtype) {
  TORCH_CHECK(t.is_cuda(), name, " must be CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.scalar_type() == dtype, name, " must be ", c10::toString(dtype), ", got ",
              c10::toString(t.scalar_type()));
}

inline void check_same_device(const torch::Tensor& a, const torch::Tensor& b, const char* an,
                              const char* bn) {
  TORCH_CHECK(a.device() == b.device(), an, " and ", bn, " must be on the same device");
}

inline void check_status(int status, const char* op) {
  TORCH_CHECK(status == CAB_OK, op, " failed: ", cab_status_string(status));
}

inline cudaStream_t current_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

template <typename T>
inline T* ptr(const torch::Tensor& t) {
  return reinterpret_cast<T*>(t.data_ptr());
}

}  // namespace cab_binding
