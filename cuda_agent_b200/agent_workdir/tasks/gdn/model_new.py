"""Gated DeltaNet decode on the CUDA extension.

Same constructor and forward signature as the eager model of this task
(forward(state, q, k, v, g, beta) -> (o, new_state)); the body is one extension
call, as in the reference's agent_workdir/model_new.py:6-13. `state` is updated
in place and returned as `new_state`.

A decode loop calls forward step after step on the same state, so the module
flips the op's walk-direction bit (config 16) from call to call: every step then
starts on the rows the previous one wrote last, which are still in L2. The
result of a call does not depend on the bit.
"""
import torch
import torch.nn as nn
import cuda_extension


class ModelNew(nn.Module):

    def __init__(self, B: int, Hq: int, Hv: int) -> None:
        super().__init__()
        self.B, self.Hq, self.Hv = B, Hq, Hv
        self.calls = 0

    def forward(self, state, q, k, v, g, beta):
        config = 16 if self.calls & 1 else 0
        self.calls += 1
        return cuda_extension.gdn_decode_forward(state, q, k, v, g, beta, config)
