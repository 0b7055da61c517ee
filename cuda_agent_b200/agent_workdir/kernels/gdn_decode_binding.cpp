// cuda_extension.gdn_decode_forward(state, q, k, v, g, beta, config=0) -> (o, state)
//
// One Gated DeltaNet decode step. `state` (fp32 [B,Hv,128,128]) is updated in
// place and returned as the second element, so the result has the same
// container shape as the eager model's `(o, new_state)`; `o` is a new fp32
// [B,Hv,128] tensor. Written in the style of the reference binding
// (agent_workdir/kernels/axpby_binding.cpp:17-44): validate, allocate the
// output, take the current stream, call the extern "C" launcher.
#include "binding_common.h"

static std::tuple<torch::Tensor, torch::Tensor> gdn_decode_forward(
    torch::Tensor state, torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor g,
    torch::Tensor beta, int config = 0) {
  using namespace cab_binding;
  check_cuda_contig(state, "state", torch::kFloat32);
  check_cuda_contig(q, "q", torch::kBFloat16);
  check_cuda_contig(k, "k", torch::kBFloat16);
  check_cuda_contig(v, "v", torch::kBFloat16);
  check_cuda_contig(g, "g", torch::kFloat32);
  check_cuda_contig(beta, "beta", torch::kFloat32);
  TORCH_CHECK(state.dim() == 4 && state.size(2) == 128 && state.size(3) == 128,
              "state must be [B, Hv, 128, 128]");
  const int64_t B = state.size(0), Hv = state.size(1);
  TORCH_CHECK(q.dim() == 3 && q.size(0) == B && q.size(2) == 128, "q must be [B, Hq, 128]");
  const int64_t Hq = q.size(1);
  TORCH_CHECK(Hq > 0 && Hv % Hq == 0, "Hv must be a multiple of Hq");
  TORCH_CHECK(k.sizes() == q.sizes(), "k must have the shape of q");
  TORCH_CHECK(v.dim() == 3 && v.size(0) == B && v.size(1) == Hv && v.size(2) == 128,
              "v must be [B, Hv, 128]");
  TORCH_CHECK(g.dim() == 2 && g.size(0) == B && g.size(1) == Hv, "g must be [B, Hv]");
  TORCH_CHECK(beta.sizes() == g.sizes(), "beta must be [B, Hv]");
  for (const torch::Tensor* t : {&q, &k, &v, &g, &beta})
    check_same_device(state, *t, "state", "every other argument");
  TORCH_CHECK(B * Hv <= INT32_MAX, "B*Hv too large");

  c10::cuda::CUDAGuard guard(state.device());
  auto out = torch::empty({B, Hv, 128}, state.options());
  check_status(
      gdn_decode_launcher(ptr<float>(state), ptr<float>(out), ptr<const cab_bf16>(q),
                          ptr<const cab_bf16>(k), ptr<const cab_bf16>(v), ptr<const float>(g),
                          ptr<const float>(beta), static_cast<int>(B), static_cast<int>(Hq),
                          static_cast<int>(Hv), config, current_stream()),
      "gdn_decode_forward");
  return {out, state};
}

static void register_gdn_decode(pybind11::module& m) {
  m.def("gdn_decode_forward", &gdn_decode_forward, py::arg("state"), py::arg("q"), py::arg("k"),
        py::arg("v"), py::arg("g"), py::arg("beta"), py::arg("config") = 0);
}

REGISTER_BINDING(gdn_decode, register_gdn_decode);
