// Python binding of the smoke-test op. Signature and checks as in the reference
// (agent_workdir/kernels/axpby_binding.cpp:17-44): cuda_extension.axpby_forward(a, b, alpha, config=0).
#include "binding_common.h"

static torch::Tensor axpby_forward(torch::Tensor a, torch::Tensor b, double alpha, int config = 0) {
  using namespace cab_binding;
  check_cuda_contig(a, "a", torch::kFloat32);
  check_cuda_contig(b, "b", torch::kFloat32);
  TORCH_CHECK(a.sizes() == b.sizes(), "a and b must have the same shape");
  check_same_device(a, b, "a", "b");
  TORCH_CHECK(a.numel() <= INT32_MAX, "axpby_forward supports at most 2^31-1 elements");
  c10::cuda::CUDAGuard guard(a.device());
  auto out = torch::empty_like(a);
  check_status(axpby_launcher(ptr<float>(out), ptr<const float>(a), ptr<const float>(b),
                              static_cast<float>(alpha), static_cast<int>(a.numel()), config,
                              current_stream()),
               "axpby_forward");
  return out;
}

static void register_axpby(pybind11::module& m) {
  m.def("axpby_forward", &axpby_forward, py::arg("a"), py::arg("b"), py::arg("alpha"),
        py::arg("config") = 0);
}

REGISTER_BINDING(axpby, register_axpby);
