"""Eager oracle for Gated DeltaNet single-step decode (TEST INFRASTRUCTURE).

Shape of the file follows the reference's eager-model slot
(agent_workdir/model.py:9-26): ``Model``, ``get_inputs()`` returning CPU tensors,
``get_init_inputs()`` returning the constructor arguments. The reference ships
no GDN model, test or golden vector, so parity of this path is UNPINNED by the
reference; the arithmetic below restates the operator definition:

    alpha = exp(g)                       per (b, hv), g <= 0
    S'    = alpha * S (I - beta k k^T) + beta v k^T
    o     = S' q / sqrt(dk)

with S stored as [B, Hv, dv, dk] (row = value channel) so that ``o = S' q``.
q and k arrive L2-normalised (the generator does it; the op does not), value
head hv uses q/k head ``hv // (Hv // Hq)``, everything is computed in fp32 from
the bf16 inputs, and ``o`` is fp32 because bf16 cannot hold rel 1e-3.

Inputs are drawn in fp32 from a module-level ``torch.Generator`` (seed 1234 +
config index) and then cast, so every consumer sees identical bits; successive
``get_inputs()`` calls continue the same stream, giving the verification loop
five different but reproducible trials.

The config is chosen with the environment variable ``CAB_GDN_CONFIG``:
``0`` -> B=4, Hq=Hv=8 (the CPU-sized case), ``1`` -> B=256, Hq=16, Hv=32.
"""
import os

import torch
import torch.nn as nn

D = 128
CONFIGS = {
    0: dict(B=4, Hq=8, Hv=8),
    1: dict(B=256, Hq=16, Hv=32),
}
CONFIG = int(os.environ.get("CAB_GDN_CONFIG", "0"))

# How utils/verification.py compares each element of the output tuple.
OUTPUT_POLICY = [("rel", 1e-3), ("rel", 1e-3)]


class Model(nn.Module):
    """One decode step. forward(state, q, k, v, g, beta) -> (o, new_state)."""

    def __init__(self, B: int, Hq: int, Hv: int) -> None:
        super().__init__()
        assert Hv % Hq == 0
        self.B, self.Hq, self.Hv = B, Hq, Hv

    def forward(self, state, q, k, v, g, beta):
        group = self.Hv // self.Hq
        qf = q.float().repeat_interleave(group, dim=1)          # [B, Hv, dk]
        kf = k.float().repeat_interleave(group, dim=1)
        vf = v.float()                                           # [B, Hv, dv]
        alpha = torch.exp(g.float())[..., None, None]            # [B, Hv, 1, 1]
        bt = beta.float()[..., None, None]
        S = state.float()
        u = torch.einsum("bhij,bhj->bhi", S, kf)                 # S k
        # alpha * S (I - beta k k^T) + beta v k^T
        S_new = alpha * (S - bt * u[..., :, None] * kf[..., None, :]) \
            + bt * vf[..., :, None] * kf[..., None, :]
        o = torch.einsum("bhij,bhj->bhi", S_new, qf) * (D ** -0.5)
        return o, S_new


_GEN = None


def _generator() -> torch.Generator:
    global _GEN
    if _GEN is None:
        _GEN = torch.Generator(device="cpu")
        _GEN.manual_seed(1234 + CONFIG)
    return _GEN


def reseed(seed=None) -> None:
    """Restart the input stream (tests call this to make a case self-contained)."""
    global _GEN
    _GEN = torch.Generator(device="cpu")
    _GEN.manual_seed(1234 + CONFIG if seed is None else seed)


def make_step_inputs(B, Hq, Hv, gen):
    """q, k, v, g, beta for one decode step (CPU tensors)."""
    q = torch.randn(B, Hq, D, generator=gen)
    k = torch.randn(B, Hq, D, generator=gen)
    q = (q / q.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
    k = (k / k.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
    v = torch.randn(B, Hv, D, generator=gen).to(torch.bfloat16)
    g = -torch.nn.functional.softplus(torch.randn(B, Hv, generator=gen))
    beta = torch.sigmoid(torch.randn(B, Hv, generator=gen))
    return q, k, v, g, beta


def make_state(B, Hv, gen):
    return torch.randn(B, Hv, D, D, generator=gen) * 0.02


def get_inputs():
    c = CONFIGS[CONFIG]
    gen = _generator()
    state = make_state(c["B"], c["Hv"], gen)
    return [state, *make_step_inputs(c["B"], c["Hq"], c["Hv"], gen)]


def get_init_inputs():
    c = CONFIGS[CONFIG]
    return [c["B"], c["Hq"], c["Hv"]]
