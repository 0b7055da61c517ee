// cuda_extension.mla_sparse_decode_forward(q, kv, seq_len, idx, softmax_scale, nsplit=0, check=False, config=0)
//   -> out bf16 [B, Sq, Hh, 512]   (q [B, Sq, Hh, 576], idx [B, Sq, topk], seq_len [B] or [B, Sq])
// cuda_extension.mla_gather_rows(kv, seq_len, idx) -> rows bf16 [B, topk, 576]
//
// nsplit = 0 picks the number of splits so that the grid covers the 148 SMs: B * Hh/64 CTAs
// per split. Written after the reference binding (agent_workdir/kernels/axpby_binding.cpp:17-44):
// validate, allocate output and scratch with torch::empty, current stream, launcher.
#include "binding_common.h"

namespace {
using cab_binding::check_cuda_contig;
using cab_binding::check_status;
using cab_binding::current_stream;
using cab_binding::ptr;

void check_inputs(const torch::Tensor& kv, const torch::Tensor& seq_len, const torch::Tensor& idx) {
  check_cuda_contig(kv, "kv", torch::kBFloat16);
  check_cuda_contig(seq_len, "seq_len", torch::kInt32);
  check_cuda_contig(idx, "idx", torch::kInt32);
  TORCH_CHECK(kv.dim() == 3 && kv.size(2) == 576, "kv must be [B, S, 576]");
  TORCH_CHECK((seq_len.dim() == 1 || (seq_len.dim() == 2 && seq_len.size(1) == idx.size(1))) &&
                  seq_len.size(0) == kv.size(0),
              "seq_len must be [B] or [B, Sq]");
  TORCH_CHECK(idx.dim() == 3 && idx.size(0) == kv.size(0) && idx.size(1) >= 1, "idx must be [B, Sq, topk]");
}

torch::Tensor mla_sparse_decode_forward(torch::Tensor q, torch::Tensor kv, torch::Tensor seq_len, torch::Tensor idx,
                                        double softmax_scale, int64_t nsplit, bool check, int config) {
  check_cuda_contig(q, "q", torch::kBFloat16);
  check_inputs(kv, seq_len, idx);
  TORCH_CHECK(q.dim() == 4 && q.size(0) == kv.size(0) && q.size(1) == idx.size(1) && q.size(3) == 576,
              "q must be [B, Sq, Hh, 576] with Sq = idx.size(1)");
  const int64_t B = q.size(0), Sq = q.size(1), Hh = q.size(2), S = kv.size(1), topk = idx.size(2);
  // one valid length per (sequence, query token); a [B] tensor applies to every token of the sequence
  if (seq_len.dim() == 1 && Sq > 1) seq_len = seq_len.unsqueeze(1).expand({B, Sq}).contiguous();
  TORCH_CHECK(Hh % 64 == 0, "the number of heads must be a multiple of 64");
  if (nsplit <= 0) {
    const int64_t ctas = B * Sq * (Hh / 64), blocks = (topk + 63) / 64;
    nsplit = std::max<int64_t>(1, std::min<int64_t>(blocks, 148 / std::max<int64_t>(ctas, 1)));
  }
  c10::cuda::CUDAGuard guard(q.device());
  auto out = torch::empty({B, Sq, Hh, 512}, q.options());
  torch::Tensor scratch, status = torch::empty({1}, q.options().dtype(torch::kInt32));
  const size_t bytes = mla_sparse_decode_scratch_bytes((int)(B * Sq), (int)Hh, (int)nsplit);
  if (bytes) scratch = torch::empty({(int64_t)bytes}, q.options().dtype(torch::kUInt8));
  check_status(mla_sparse_decode_multi_launcher(ptr<cab_bf16>(out), ptr<const cab_bf16>(q), ptr<const cab_bf16>(kv),
                                                ptr<const int>(seq_len), ptr<const int>(idx), (int)B, (int)Sq, (int)Hh,
                                                (int)S, (int)topk, (float)softmax_scale, (int)nsplit,
                                                bytes ? scratch.data_ptr() : nullptr, ptr<int>(status), config,
                                                current_stream()),
               "mla_sparse_decode_forward");
  if (check) TORCH_CHECK(status.item<int>() == 0, "mla_sparse_decode: a bounded wait gave up (code ", status.item<int>(), ")");
  return out;
}

torch::Tensor mla_gather_rows(torch::Tensor kv, torch::Tensor seq_len, torch::Tensor idx) {
  check_inputs(kv, seq_len, idx);
  TORCH_CHECK(idx.size(1) == 1 && seq_len.dim() == 1, "mla_gather_rows takes idx [B, 1, topk] and seq_len [B]");
  c10::cuda::CUDAGuard guard(kv.device());
  auto rows = torch::empty({kv.size(0), idx.size(2), 576}, kv.options());
  check_status(mla_gather_rows_launcher(ptr<cab_bf16>(rows), ptr<const cab_bf16>(kv), ptr<const int>(seq_len),
                                        ptr<const int>(idx), (int)kv.size(0), (int)kv.size(1), (int)idx.size(2), 0,
                                        current_stream()),
               "mla_gather_rows");
  return rows;
}

void register_mla(pybind11::module& m) {
  m.def("mla_sparse_decode_forward", &mla_sparse_decode_forward, py::arg("q"), py::arg("kv"), py::arg("seq_len"),
        py::arg("idx"), py::arg("softmax_scale"), py::arg("nsplit") = 0, py::arg("check") = false,
        py::arg("config") = 0);
  m.def("mla_gather_rows", &mla_gather_rows, py::arg("kv"), py::arg("seq_len"), py::arg("idx"));
}
}  // namespace

REGISTER_BINDING(mla, register_mla);
