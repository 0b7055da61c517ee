"""Eager oracle for top-k sparse MLA decode attention (TEST INFRASTRUCTURE).

File shape follows the reference's eager-model slot (agent_workdir/model.py:9-26).
The reference ships no attention model, test or vector, so parity of this path is
UNPINNED by the reference; this file restates the operator definition and the
tests pin it with float64 loops and hand cases.

Absorbed multi-head latent attention, one new token per sequence:

  q        bf16 [B, 1, Hh, 576]      (512 latent + 64 rope dims)
  kv       bf16 [B, S, 576]          latent KV cache, one row per cached token
  seq_len  int32 [B]                 valid rows of each sequence
  idx      int32 [B, 1, topk]        selected rows (shared by all heads), unsorted;
                                     an entry is valid iff 0 <= idx < seq_len[b]
  scores   = (q . kv[b, idx]^T) * scale          fp32, scale = 1/sqrt(192)
  p        = softmax over the VALID entries      fp32
  out      = p . kv[b, idx][:, :512]             fp32 -> bf16   [B, 1, Hh, 512]
  a query with no valid entry yields zeros.
Several query tokens per sequence (speculative / multi-token decode): q [B, Sq, Hh, 576],
idx [B, Sq, topk], seq_len [B] or [B, Sq]; every token is the one-token operator on the
shared cache with its own selection and valid length.

``gather_rows`` is the index-validation + row-gather step on its own (invalid
entries give zero rows); it is compared bit for bit.

``CAB_MLA_CONFIG``: 0 = CPU-sized (B=3, 16 heads, S=300, topk=64);
1 = B=3, 64 heads, S=600, topk=320 (the smallest head count the CUDA operator takes);
2 = B=64, 128 heads, S=32768, topk=2048, lengths uniform in [8192, 32768].
"""
import os

import torch
import torch.nn as nn

D_QK, D_V = 576, 512
SCALE = 192 ** -0.5
CONFIGS = {
    0: dict(B=3, Hh=16, S=300, topk=64, min_len=40),
    1: dict(B=3, Hh=64, S=600, topk=320, min_len=200),
    2: dict(B=64, Hh=128, S=32768, topk=2048, min_len=8192),
}
CONFIG = int(os.environ.get("CAB_MLA_CONFIG", "0"))

OUTPUT_POLICY = ("atol", 2e-2)


def valid_mask(idx: torch.Tensor, seq_len: torch.Tensor) -> torch.Tensor:
    """[B, topk] bool."""
    i = idx[:, 0, :].long()
    return (i >= 0) & (i < seq_len.long()[:, None])


def gather_rows(kv: torch.Tensor, idx: torch.Tensor, seq_len: torch.Tensor) -> torch.Tensor:
    """[B, topk, 576] bf16: the selected rows, zero where the entry is invalid."""
    ok = valid_mask(idx, seq_len)
    safe = torch.where(ok, idx[:, 0, :].long(), torch.zeros_like(idx[:, 0, :].long()))
    rows = torch.gather(kv, 1, safe[..., None].expand(-1, -1, kv.shape[-1]))
    return torch.where(ok[..., None], rows, torch.zeros_like(rows))


class Model(nn.Module):
    """forward(q, kv, seq_len, idx) -> out bf16 [B, Sq, Hh, 512].

    Sq = q.shape[1] query tokens per sequence (1 in the configs): token s of sequence b uses
    idx[b, s] and the valid length seq_len[b, s] (a [B] seq_len applies to every token)."""

    def __init__(self, B: int, Hh: int, S: int, topk: int) -> None:
        super().__init__()
        self.B, self.Hh, self.S, self.topk = B, Hh, S, topk

    @staticmethod
    def one_token(q, kv, seq_len, idx):
        """q [B, Hh, 576], seq_len [B], idx [B, 1, topk] -> fp32 [B, Hh, 512]."""
        ok = valid_mask(idx, seq_len)                                   # [B, topk]
        rows = gather_rows(kv, idx, seq_len).float()                    # [B, topk, 576]
        scores = torch.einsum("bhd,btd->bht", q.float(), rows) * SCALE
        scores = scores.masked_fill(~ok[:, None, :], float("-inf"))
        p = torch.softmax(scores, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)                                # rows with no valid entry
        return torch.einsum("bht,btd->bhd", p, rows[..., :D_V])

    def forward(self, q, kv, seq_len, idx):
        outs = []
        for s in range(q.shape[1]):
            lens = seq_len if seq_len.dim() == 1 else seq_len[:, s]
            outs.append(self.one_token(q[:, s], kv, lens, idx[:, s:s + 1]))
        return torch.stack(outs, dim=1).to(torch.bfloat16)


_GEN = None


def reseed(seed=None) -> None:
    global _GEN
    _GEN = torch.Generator().manual_seed(1234 + CONFIG if seed is None else seed)


def make_inputs(B, Hh, S, topk, min_len, gen):
    q = torch.randn(B, 1, Hh, D_QK, generator=gen).to(torch.bfloat16)
    kv = torch.empty(B, S, D_QK, dtype=torch.bfloat16)
    for b in range(B):                                                  # keeps the fp32 staging small
        kv[b] = torch.randn(S, D_QK, generator=gen).to(torch.bfloat16)
    seq_len = torch.randint(min_len, S + 1, (B,), generator=gen, dtype=torch.int32)
    idx = torch.full((B, 1, topk), -1, dtype=torch.int32)
    for b in range(B):
        n = int(seq_len[b])
        chosen = torch.randperm(n, generator=gen)[:topk].to(torch.int32)
        idx[b, 0, : chosen.numel()] = chosen
    return [q, kv, seq_len, idx]


def get_inputs():
    if _GEN is None:
        reseed()
    c = CONFIGS[CONFIG]
    return make_inputs(c["B"], c["Hh"], c["S"], c["topk"], c["min_len"], _GEN)


def get_init_inputs():
    c = CONFIGS[CONFIG]
    return [c["B"], c["Hh"], c["S"], c["topk"]]
