"""Writes tests/golden/mla_small.npz and tests/golden/moe_config{0,1}.npz from the eager oracles.

Run from the repository root:  python tests/golden/make_mla_moe_golden.py
The reference ships no vector for these operators, so the fixtures pin the oracles against themselves
over time (an edit of an oracle that changes its results fails the CPU tests) and give the GPU tests a
file-based expectation that does not depend on running the oracle. Inputs are not stored: they are
regenerated from the seeds below by the same functions the tests call.

  mla_small.npz     sparse MLA decode, 2 sequences x 64 heads and 2 x 128 heads, 128 of 300 rows, seed 1:
                    every third element of the flattened bf16 outputs, as uint16
  moe_config{c}.npz FP8 MoE layer, CAB_MOE_CONFIG c, get_inputs() after reseed(): routing indices (int32),
                    routing weights (fp32) and the bf16 output as uint16
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "tests"))
from conftest import load_oracle  # noqa: E402

HERE = Path(__file__).resolve().parent
MLA_STRIDE = 3


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def mla_case(m, heads):
    gen = torch.Generator().manual_seed(1)
    q, kv, seq_len, idx = m.make_inputs(2, heads, 300, 128, 40, gen)
    idx[0, 0, 3] = -1
    idx[1, 0, 64] = 10 ** 6
    return q, kv, seq_len, idx


def main():
    torch.set_num_threads(1)
    m = load_oracle("mla", {"CAB_MLA_CONFIG": 0})
    outs = {}
    with torch.no_grad():
        for heads in (64, 128):
            q, kv, seq_len, idx = mla_case(m, heads)
            outs[f"out{heads}"] = bits(m.Model(2, heads, 300, 128)(q, kv, seq_len, idx)).reshape(-1)[::MLA_STRIDE]
    np.savez_compressed(HERE / "mla_small.npz", seed=np.int64(1), stride=np.int64(MLA_STRIDE), **outs)
    print("wrote mla_small.npz", (HERE / "mla_small.npz").stat().st_size, "bytes")
    for cfg in (0, 1):
        m = load_oracle("moe", {"CAB_MOE_CONFIG": cfg})
        m.reseed()
        (x,) = m.get_inputs()
        model = m.Model(*m.get_init_inputs())
        with torch.no_grad():
            idx, w = model.route(model.logits(x))
            out = model(x)
        path = HERE / f"moe_config{cfg}.npz"
        np.savez_compressed(path, idx=idx.numpy().astype(np.int32), w=w.numpy().astype(np.float32), out=bits(out))
        print("wrote", path.name, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
