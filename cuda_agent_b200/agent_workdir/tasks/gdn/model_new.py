"""Gated DeltaNet decode on the CUDA extension.

Same constructor and forward signature as the eager model of this task
(forward(state, q, k, v, g, beta) -> (o, new_state)); the body is one extension
call, as in the reference's agent_workdir/model_new.py:6-13. `state` is updated
in place and returned as `new_state`.
"""
import torch
import torch.nn as nn
import cuda_extension


class ModelNew(nn.Module):

    def __init__(self, B: int, Hq: int, Hv: int) -> None:
        super().__init__()
        self.B, self.Hq, self.Hv = B, Hq, Hv

    def forward(self, state, q, k, v, g, beta):
        return cuda_extension.gdn_decode_forward(state, q, k, v, g, beta, 0)
