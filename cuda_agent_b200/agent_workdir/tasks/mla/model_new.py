"""Top-k sparse MLA decode attention on the CUDA extension.

Same constructor and forward signature as the eager model of this task
(forward(q, kv, seq_len, idx) -> out bf16 [B, 1, Hh, 512]); one extension call,
as in the reference's agent_workdir/model_new.py:12-13.
"""
import torch
import torch.nn as nn
import cuda_extension


class ModelNew(nn.Module):

    def __init__(self, B: int, Hh: int, S: int, topk: int) -> None:
        super().__init__()
        self.B, self.Hh, self.S, self.topk = B, Hh, S, topk
        self.softmax_scale = 192 ** -0.5

    def forward(self, q, kv, seq_len, idx):
        return cuda_extension.mla_sparse_decode_forward(q, kv, seq_len, idx, self.softmax_scale, 0, False, 0)
