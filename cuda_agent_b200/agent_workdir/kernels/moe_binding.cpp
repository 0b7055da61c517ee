// cuda_extension.moe_forward / moe_route: the FP8 block-scaled MoE layer.
//
//   moe_route(x, router_w, router_bias, k, routing, n_group, topk_group, scaling)
//       -> (topk_idx int32 [T,k], topk_w fp32 [T,k])
//   moe_forward(x, router_w, router_bias, w13_q, w13_s, w2_q, w2_s,
//               shared_w13_q, shared_w13_s, shared_w2_q, shared_w2_s,
//               k, routing, n_group, topk_group, scaling, check, config) -> out bf16 [T,H]
//
// routing: 0 = softmax top-k, 1 = sigmoid + bias with group restriction. The shared_*
// tensors may be None (no shared expert). `check` = True synchronises and raises if a
// kernel reported a failed bounded wait or a bad expert id. The wrapper follows the
// reference binding's pattern (agent_workdir/kernels/axpby_binding.cpp:17-44): validate,
// allocate outputs and scratch with torch::empty, take the current stream, call the
// extern "C" launchers in order. Nothing synchronises unless `check` is set.
#include "binding_common.h"

#include <optional>

namespace {
using cab_binding::check_cuda_contig;
using cab_binding::check_status;
using cab_binding::current_stream;
using cab_binding::ptr;
using OptTensor = std::optional<torch::Tensor>;

struct Routed {
  torch::Tensor idx, w;
};

Routed route(const torch::Tensor& x, const torch::Tensor& router_w, const torch::Tensor& router_bias,
             int64_t k, int64_t routing, int64_t n_group, int64_t topk_group, double scaling,
             cudaStream_t stream) {
  const int64_t T = x.size(0), H = x.size(1), E = router_w.size(0);
  auto f32 = x.options().dtype(torch::kFloat32);
  auto logits = torch::empty({T, E}, f32);
  check_status(moe_router_logits_launcher(ptr<float>(logits), ptr<const cab_bf16>(x),
                                          ptr<const cab_bf16>(router_w), (int)T, (int)H, (int)E, 0, stream),
               "moe_router_logits");
  Routed r{torch::empty({T, k}, x.options().dtype(torch::kInt32)), torch::empty({T, k}, f32)};
  if (routing == 0) {
    check_status(moe_route_softmax_topk_launcher(ptr<int>(r.idx), ptr<float>(r.w), ptr<const float>(logits),
                                                 (int)T, (int)E, (int)k, 0, stream),
                 "moe_route_softmax_topk");
  } else {
    check_status(moe_route_sigmoid_group_topk_launcher(ptr<int>(r.idx), ptr<float>(r.w), ptr<const float>(logits),
                                                       ptr<const float>(router_bias), (int)T, (int)E, (int)k,
                                                       (int)n_group, (int)topk_group, (float)scaling, 0, stream),
                 "moe_route_sigmoid_group_topk");
  }
  return r;
}

void check_router_args(const torch::Tensor& x, const torch::Tensor& router_w, const torch::Tensor& router_bias) {
  check_cuda_contig(x, "x", torch::kBFloat16);
  check_cuda_contig(router_w, "router_w", torch::kBFloat16);
  check_cuda_contig(router_bias, "router_bias", torch::kFloat32);
  TORCH_CHECK(x.dim() == 2 && router_w.dim() == 2 && router_w.size(1) == x.size(1), "x [T,H], router_w [E,H]");
  TORCH_CHECK(router_bias.numel() == router_w.size(0), "router_bias must be [E]");
}

void check_expert_weights(const torch::Tensor& w13_q, const torch::Tensor& w13_s, const torch::Tensor& w2_q,
                          const torch::Tensor& w2_s, int64_t E, int64_t H, int64_t& I, const char* what) {
  check_cuda_contig(w13_q, what, at::kFloat8_e4m3fn);
  check_cuda_contig(w2_q, what, at::kFloat8_e4m3fn);
  check_cuda_contig(w13_s, what, torch::kFloat32);
  check_cuda_contig(w2_s, what, torch::kFloat32);
  TORCH_CHECK(w2_q.numel() == E * H * (w2_q.size(-1)) && w2_q.size(-2) == H, what, ": w2 must be [E,H,I]");
  I = w2_q.size(-1);
  TORCH_CHECK(w13_q.size(-1) == H && w13_q.size(-2) == 2 * I && w13_q.numel() == E * 2 * I * H, what,
              ": w13 must be [E,2I,H]");
  TORCH_CHECK(w13_s.numel() == E * (2 * I / 128) * (H / 128) && w2_s.numel() == E * (H / 128) * (I / 128), what,
              ": scale tensors must be [E,2I/128,H/128] and [E,H/128,I/128]");
  TORCH_CHECK(H % 256 == 0 && I % 128 == 0, "H must be a multiple of 256 and I of 128");
}

std::tuple<torch::Tensor, torch::Tensor> moe_route(torch::Tensor x, torch::Tensor router_w,
                                                   torch::Tensor router_bias, int64_t k, int64_t routing,
                                                   int64_t n_group, int64_t topk_group, double scaling) {
  check_router_args(x, router_w, router_bias);
  c10::cuda::CUDAGuard guard(x.device());
  Routed r = route(x, router_w, router_bias, k, routing, n_group, topk_group, scaling, current_stream());
  return {r.idx, r.w};
}

torch::Tensor moe_forward(torch::Tensor x, torch::Tensor router_w, torch::Tensor router_bias,
                          torch::Tensor w13_q, torch::Tensor w13_s, torch::Tensor w2_q, torch::Tensor w2_s,
                          OptTensor shared_w13_q, OptTensor shared_w13_s, OptTensor shared_w2_q,
                          OptTensor shared_w2_s, int64_t k, int64_t routing, int64_t n_group,
                          int64_t topk_group, double scaling, bool check, int config) {
  check_router_args(x, router_w, router_bias);
  const int64_t T = x.size(0), H = x.size(1), E = router_w.size(0);
  int64_t I = 0;
  check_expert_weights(w13_q, w13_s, w2_q, w2_s, E, H, I, "expert weights");
  const bool has_shared = shared_w13_q.has_value();
  if (has_shared) {
    TORCH_CHECK(shared_w13_s && shared_w2_q && shared_w2_s, "all four shared-expert tensors or none");
    int64_t Is = 0;
    check_expert_weights(*shared_w13_q, *shared_w13_s, *shared_w2_q, *shared_w2_s, 1, H, Is, "shared expert");
  }
  c10::cuda::CUDAGuard guard(x.device());
  cudaStream_t stream = current_stream();
  auto i32 = x.options().dtype(torch::kInt32);
  auto f32 = x.options().dtype(torch::kFloat32);
  auto u8 = x.options().dtype(torch::kUInt8);

  Routed r = route(x, router_w, router_bias, k, routing, n_group, topk_group, scaling, stream);

  // permutation tables and the padded row space
  const int max_tiles = moe_permute_max_tiles((int)T, (int)k, (int)E);
  const int64_t cap = (int64_t)max_tiles * 128;
  auto tables = torch::empty({3 * (E + 1) + 3 * T * k + max_tiles + 1 + 2}, i32);
  int* base = ptr<int>(tables);
  int* counts = base;
  int* offsets = counts + (E + 1);
  int* pad_offsets = offsets + (E + 1);
  int* perm = pad_offsets + (E + 1);
  int* inv_perm = perm + T * k;
  int* dst_row = inv_perm + T * k;
  int* tile_expert = dst_row + T * k;
  int* num_tiles = tile_expert + max_tiles;
  int* status = num_tiles + 1;  // two ints: one per GEMM
  auto scratch = torch::empty({(int64_t)moe_permute_scratch_bytes((int)T, (int)k, (int)E)}, u8);
  check_status(moe_permute_launcher(ptr<const int>(r.idx), (int)T, (int)k, (int)E, counts, offsets, pad_offsets,
                                    perm, inv_perm, dst_row, tile_expert, num_tiles, max_tiles,
                                    scratch.data_ptr(), 0, stream),
               "moe_permute");

  auto a_q = torch::empty({cap, H}, u8);
  auto a_s = torch::empty({H / 128, cap}, f32);
  check_status(moe_quant_dispatch_launcher(ptr<cab_e4m3>(a_q), ptr<float>(a_s), ptr<const cab_bf16>(x), dst_row,
                                           (int)T, (int)H, (int)k, (int)cap, 0, stream),
               "moe_quant_dispatch");
  auto h_q = torch::empty({cap, I}, u8);
  auto h_s = torch::empty({I / 128, cap}, f32);
  auto y = torch::empty({cap, H}, x.options());
  check_status(moe_grouped_gemm_fp8_launcher(0, h_q.data_ptr(), ptr<float>(h_s), ptr<const cab_e4m3>(a_q),
                                             ptr<const float>(a_s), ptr<const cab_e4m3>(w13_q),
                                             ptr<const float>(w13_s), tile_expert, num_tiles, max_tiles, (int)cap,
                                             (int)cap, (int)E, (int)I, (int)H, status, config, stream),
               "moe_grouped_gemm_fp8 (gate/up)");
  check_status(moe_grouped_gemm_fp8_launcher(1, y.data_ptr(), nullptr, ptr<const cab_e4m3>(h_q),
                                             ptr<const float>(h_s), ptr<const cab_e4m3>(w2_q),
                                             ptr<const float>(w2_s), tile_expert, num_tiles, max_tiles, (int)cap,
                                             (int)cap, (int)E, (int)H, (int)I, status + 1, config, stream),
               "moe_grouped_gemm_fp8 (down)");

  torch::Tensor y_shared;
  torch::Tensor shared_status;
  if (has_shared) {
    const int64_t Is = shared_w2_q->size(-1);
    const int tiles = (int)((T + 127) / 128);
    const int64_t scap = (int64_t)tiles * 128;
    auto xs_q = torch::empty({scap, H}, u8);
    auto xs_s = torch::empty({H / 128, scap}, f32);
    check_status(moe_quant_dispatch_launcher(ptr<cab_e4m3>(xs_q), ptr<float>(xs_s), ptr<const cab_bf16>(x), nullptr,
                                             (int)T, (int)H, 1, (int)scap, 0, stream),
                 "moe_quant_dispatch (shared)");
    auto hs_q = torch::empty({scap, Is}, u8);
    auto hs_s = torch::empty({Is / 128, scap}, f32);
    y_shared = torch::empty({scap, H}, x.options());
    shared_status = torch::empty({2}, i32);
    check_status(moe_grouped_gemm_fp8_launcher(0, hs_q.data_ptr(), ptr<float>(hs_s), ptr<const cab_e4m3>(xs_q),
                                               ptr<const float>(xs_s), ptr<const cab_e4m3>(*shared_w13_q),
                                               ptr<const float>(*shared_w13_s), nullptr, nullptr, tiles, (int)scap,
                                               (int)scap, 1, (int)Is, (int)H, ptr<int>(shared_status), config,
                                               stream),
                 "moe_grouped_gemm_fp8 (shared gate/up)");
    check_status(moe_grouped_gemm_fp8_launcher(1, y_shared.data_ptr(), nullptr, ptr<const cab_e4m3>(hs_q),
                                               ptr<const float>(hs_s), ptr<const cab_e4m3>(*shared_w2_q),
                                               ptr<const float>(*shared_w2_s), nullptr, nullptr, tiles, (int)scap,
                                               (int)scap, 1, (int)H, (int)Is, ptr<int>(shared_status) + 1, config,
                                               stream),
                 "moe_grouped_gemm_fp8 (shared down)");
  }

  auto out = torch::empty({T, H}, x.options());
  check_status(moe_combine_launcher(ptr<cab_bf16>(out), ptr<const cab_bf16>(y), dst_row, ptr<const float>(r.w),
                                    has_shared ? ptr<const cab_bf16>(y_shared) : nullptr, (int)T, (int)H, (int)k,
                                    0, stream),
               "moe_combine");
  if (check) {
    auto st = tables.slice(0, tables.numel() - 2).cpu();
    TORCH_CHECK(st[0].item<int>() == 0 && st[1].item<int>() == 0, "moe_forward: a GEMM kernel gave up a bounded wait (codes ",
                st[0].item<int>(), ", ", st[1].item<int>(), ")");
    auto flag = scratch.cpu();
    const int permute_flag = reinterpret_cast<const int*>(flag.data_ptr<uint8_t>())[flag.numel() / 4 - 1];
    TORCH_CHECK(permute_flag == 0, "moe_forward: permutation flagged code ", permute_flag);
    if (has_shared) {
      auto ss = shared_status.cpu();
      TORCH_CHECK(ss[0].item<int>() == 0 && ss[1].item<int>() == 0, "moe_forward: shared-expert GEMM gave up a wait");
    }
  }
  return out;
}

void register_moe(pybind11::module& m) {
  m.def("moe_route", &moe_route, py::arg("x"), py::arg("router_w"), py::arg("router_bias"), py::arg("k"),
        py::arg("routing") = 0, py::arg("n_group") = 1, py::arg("topk_group") = 1, py::arg("scaling") = 1.0);
  m.def("moe_forward", &moe_forward, py::arg("x"), py::arg("router_w"), py::arg("router_bias"), py::arg("w13_q"),
        py::arg("w13_s"), py::arg("w2_q"), py::arg("w2_s"), py::arg("shared_w13_q") = py::none(),
        py::arg("shared_w13_s") = py::none(), py::arg("shared_w2_q") = py::none(),
        py::arg("shared_w2_s") = py::none(), py::arg("k") = 1, py::arg("routing") = 0, py::arg("n_group") = 1,
        py::arg("topk_group") = 1, py::arg("scaling") = 1.0, py::arg("check") = false, py::arg("config") = 0);
}
}  // namespace

REGISTER_BINDING(moe, register_moe);
