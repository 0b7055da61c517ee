// cuda_extension.moe_ep_*: the expert-parallel FP8 MoE layer (one process per GPU, experts in
// contiguous blocks of E / world per rank) whose dispatch and return are done by the kernels over
// peer memory. The communicator state lives in the extension, as an opaque handle:
//
//   h = moe_ep_create(rank, world, t_cap, H, k, e_local)     allocates this rank's exchange buffer
//   moe_ep_export(h) -> bytes (64)                           the buffer's CUDA IPC handle
//   moe_ep_connect(h, [bytes] * world)                       maps every other rank's buffer
//   moe_ep_connect_local([h0, h1, ...])                      the same for ranks of one process
//   moe_ep_forward(h, x, router_w, router_bias, w13_q, w13_s, w2_q, w2_s, shared_w13_q, shared_w13_s,
//                  shared_w2_q, shared_w2_s, routing, n_group, topk_group, scaling, entry_cap, check,
//                  config) -> out bf16 [T, H]
//   moe_ep_status(h) -> [8 ints]        blocking; zeros when nothing gave up (after at least one forward)
//   moe_ep_destroy(h)
//
// entry_cap = (token, expert) entries this rank accepts per call (0: all of them on one rank, 1.5 x the
// balanced share t_cap * k otherwise); what does not fit is dropped and flagged in status word 4.
// w13_* / w2_* are THIS rank's experts ([e_local, ...]); the router and the shared expert are the same
// on every rank. The wrapper follows the reference binding's pattern (agent_workdir/kernels/
// axpby_binding.cpp:17-44): validate, allocate with torch::empty (the output, and once per handle the
// workspace), take the current stream, call the extern "C" launcher. Handing the 64-byte handles from
// rank to rank is the caller's job (any transport: torch.distributed, a file, MPI).
#include "binding_common.h"

#include <map>
#include <mutex>
#include <optional>

namespace {
using cab_binding::check_cuda_contig;
using cab_binding::check_status;
using cab_binding::current_stream;
using cab_binding::ptr;
using OptTensor = std::optional<torch::Tensor>;

struct Handle {
  void* ctx = nullptr;
  torch::Tensor workspace;
  cab_moe_ep_layer_args args{};
  bool ran = false;
  int H = 0, k = 0, e_local = 0, world = 0, t_cap = 0;
};
std::mutex g_mu;
std::map<int64_t, Handle> g_handles;
int64_t g_next = 1;

Handle& lookup(int64_t h) {
  auto it = g_handles.find(h);
  TORCH_CHECK(it != g_handles.end(), "moe_ep: unknown handle ", h);
  return it->second;
}

int64_t moe_ep_create(int64_t rank, int64_t world, int64_t t_cap, int64_t H, int64_t k, int64_t e_local) {
  std::lock_guard<std::mutex> lock(g_mu);
  Handle hd;
  check_status(moe_ep_peer_create(&hd.ctx, (int)rank, (int)world, (int)t_cap, (int)H, (int)k, (int)e_local),
               "moe_ep_peer_create");
  hd.H = (int)H; hd.k = (int)k; hd.e_local = (int)e_local; hd.world = (int)world; hd.t_cap = (int)t_cap;
  const int64_t id = g_next++;
  g_handles[id] = hd;
  return id;
}

py::bytes moe_ep_export(int64_t h) {
  std::lock_guard<std::mutex> lock(g_mu);
  char buf[64];
  check_status(moe_ep_peer_export(lookup(h).ctx, buf), "moe_ep_peer_export");
  return py::bytes(buf, 64);
}

void moe_ep_connect(int64_t h, std::vector<std::string> handles) {
  std::lock_guard<std::mutex> lock(g_mu);
  Handle& hd = lookup(h);
  TORCH_CHECK((int)handles.size() == hd.world, "moe_ep_connect: one handle per rank, in rank order");
  std::string all;
  for (const auto& s : handles) {
    TORCH_CHECK(s.size() == 64, "moe_ep_connect: every handle is 64 bytes");
    all += s;
  }
  check_status(moe_ep_peer_connect_ipc(hd.ctx, all.data()), "moe_ep_peer_connect_ipc");
}

void moe_ep_connect_local(std::vector<int64_t> hs) {
  std::lock_guard<std::mutex> lock(g_mu);
  std::vector<void*> table;
  for (int64_t h : hs) table.push_back(lookup(h).ctx);
  for (int64_t h : hs) check_status(moe_ep_peer_connect_local(lookup(h).ctx, table.data()), "moe_ep_peer_connect_local");
}

torch::Tensor moe_ep_forward(int64_t h, torch::Tensor x, torch::Tensor router_w, torch::Tensor router_bias,
                             torch::Tensor w13_q, torch::Tensor w13_s, torch::Tensor w2_q, torch::Tensor w2_s,
                             OptTensor shared_w13_q, OptTensor shared_w13_s, OptTensor shared_w2_q,
                             OptTensor shared_w2_s, int64_t routing, int64_t n_group, int64_t topk_group,
                             double scaling, int64_t entry_cap, bool check, int config) {
  std::lock_guard<std::mutex> lock(g_mu);
  Handle& hd = lookup(h);
  check_cuda_contig(x, "x", torch::kBFloat16);
  check_cuda_contig(router_w, "router_w", torch::kBFloat16);
  check_cuda_contig(router_bias, "router_bias", torch::kFloat32);
  check_cuda_contig(w13_q, "w13_q", at::kFloat8_e4m3fn);
  check_cuda_contig(w2_q, "w2_q", at::kFloat8_e4m3fn);
  check_cuda_contig(w13_s, "w13_s", torch::kFloat32);
  check_cuda_contig(w2_s, "w2_s", torch::kFloat32);
  TORCH_CHECK(x.dim() == 2 && x.size(1) == hd.H, "x must be [T, H] with the H of moe_ep_create");
  const int64_t T = x.size(0), H = hd.H, E = router_w.size(0);
  TORCH_CHECK(router_w.dim() == 2 && router_w.size(1) == H && router_bias.numel() == E, "router_w [E,H], router_bias [E]");
  TORCH_CHECK(E == (int64_t)hd.e_local * hd.world, "router_w must cover e_local * world experts");
  TORCH_CHECK(w2_q.dim() == 3 && w2_q.size(0) == hd.e_local && w2_q.size(1) == H, "w2_q must be [e_local, H, I]");
  const int64_t I = w2_q.size(2);
  TORCH_CHECK(I % 128 == 0, "I must be a multiple of 128");
  TORCH_CHECK(w13_q.numel() == (int64_t)hd.e_local * 2 * I * H && w13_s.numel() == (int64_t)hd.e_local * (2 * I / 128) * (H / 128) &&
                  w2_s.numel() == (int64_t)hd.e_local * (H / 128) * (I / 128),
              "expert weights: w13_q [e_local,2I,H], w13_s [e_local,2I/128,H/128], w2_s [e_local,H/128,I/128]");
  const bool has_shared = shared_w13_q.has_value();
  if (has_shared) {
    TORCH_CHECK(shared_w13_s && shared_w2_q && shared_w2_s, "all four shared-expert tensors or none");
    check_cuda_contig(*shared_w13_q, "shared_w13_q", at::kFloat8_e4m3fn);
    check_cuda_contig(*shared_w2_q, "shared_w2_q", at::kFloat8_e4m3fn);
    check_cuda_contig(*shared_w13_s, "shared_w13_s", torch::kFloat32);
    check_cuda_contig(*shared_w2_s, "shared_w2_s", torch::kFloat32);
    TORCH_CHECK(shared_w13_q->numel() == 2 * I * H && shared_w2_q->numel() == H * I, "shared expert: [2I,H] and [H,I]");
  }
  c10::cuda::CUDAGuard guard(x.device());
  cab_moe_ep_layer_args a{};
  a.router_w = ptr<const cab_bf16>(router_w); a.router_bias = ptr<const float>(router_bias);
  a.w13_q = ptr<const cab_e4m3>(w13_q); a.w13_s = ptr<const float>(w13_s);
  a.w2_q = ptr<const cab_e4m3>(w2_q); a.w2_s = ptr<const float>(w2_s);
  if (has_shared) {
    a.shared_w13_q = ptr<const cab_e4m3>(*shared_w13_q); a.shared_w13_s = ptr<const float>(*shared_w13_s);
    a.shared_w2_q = ptr<const cab_e4m3>(*shared_w2_q); a.shared_w2_s = ptr<const float>(*shared_w2_s);
  }
  a.E = (int)E; a.I = (int)I; a.routing = (int)routing; a.n_group = (int)n_group; a.topk_group = (int)topk_group;
  // entry_cap 0: every entry when alone, 1.5 x the balanced share of t_cap * k entries otherwise
  const int64_t balanced = (int64_t)hd.t_cap * hd.k;
  if (entry_cap <= 0) entry_cap = hd.world == 1 ? balanced : balanced * 3 / 2;
  TORCH_CHECK(entry_cap <= (int64_t)hd.world * balanced, "entry_cap exceeds world * t_cap * k");
  a.scaling = (float)scaling; a.entry_cap = (int)entry_cap; a.gemm_ctas = 0;
  const size_t need = moe_ep_peer_workspace_bytes(hd.ctx, &a);
  TORCH_CHECK(need > 0, "moe_ep_forward: the layer's shapes or routing arguments were rejected");
  if (!hd.workspace.defined() || (size_t)hd.workspace.numel() < need || hd.workspace.device() != x.device())
    hd.workspace = torch::empty({(int64_t)need}, x.options().dtype(torch::kUInt8));
  hd.args = a;
  auto out = torch::empty({T, H}, x.options());
  check_status(moe_ep_peer_layer_launcher(hd.ctx, ptr<cab_bf16>(out), ptr<const cab_bf16>(x), (int)T, &a,
                                          hd.workspace.data_ptr(), (size_t)hd.workspace.numel(), config,
                                          current_stream()),
               "moe_ep_peer_layer");
  hd.ran = true;
  if (check && (config & 7) == 0) {
    int st[8];
    check_status(moe_ep_peer_read_status(hd.ctx, &hd.args, hd.workspace.data_ptr(), st), "moe_ep_peer_read_status");
    for (int i = 0; i < 8; ++i)
      TORCH_CHECK(st[i] == 0, "moe_ep_forward: status word ", i, " = ", st[i],
                  " (0-3 GEMM waits, 4 permutation, 5 wait for dispatches, 6 wait for returns)");
  }
  return out;
}

std::vector<int> moe_ep_status(int64_t h) {
  std::lock_guard<std::mutex> lock(g_mu);
  Handle& hd = lookup(h);
  std::vector<int> st(8, 0);
  if (!hd.ran) return st;
  check_status(moe_ep_peer_read_status(hd.ctx, &hd.args, hd.workspace.data_ptr(), st.data()), "moe_ep_peer_read_status");
  return st;
}

void moe_ep_destroy(int64_t h) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_handles.find(h);
  if (it == g_handles.end()) return;
  moe_ep_peer_destroy(it->second.ctx);
  g_handles.erase(it);
}

void register_moe_ep(pybind11::module& m) {
  m.def("moe_ep_create", &moe_ep_create, py::arg("rank"), py::arg("world"), py::arg("t_cap"), py::arg("H"),
        py::arg("k"), py::arg("e_local"));
  m.def("moe_ep_export", &moe_ep_export, py::arg("handle"));
  m.def("moe_ep_connect", &moe_ep_connect, py::arg("handle"), py::arg("handles"));
  m.def("moe_ep_connect_local", &moe_ep_connect_local, py::arg("handles"));
  m.def("moe_ep_forward", &moe_ep_forward, py::arg("handle"), py::arg("x"), py::arg("router_w"),
        py::arg("router_bias"), py::arg("w13_q"), py::arg("w13_s"), py::arg("w2_q"), py::arg("w2_s"),
        py::arg("shared_w13_q") = py::none(), py::arg("shared_w13_s") = py::none(),
        py::arg("shared_w2_q") = py::none(), py::arg("shared_w2_s") = py::none(), py::arg("routing") = 1,
        py::arg("n_group") = 1, py::arg("topk_group") = 1, py::arg("scaling") = 1.0, py::arg("entry_cap") = 0,
        py::arg("check") = false, py::arg("config") = 0);
  m.def("moe_ep_status", &moe_ep_status, py::arg("handle"));
  m.def("moe_ep_destroy", &moe_ep_destroy, py::arg("handle"));
}
}  // namespace

REGISTER_BINDING(moe_ep, register_moe_ep);
