"""Writes tests/golden/gdn_config0.npz from the eager oracle (oracle/gdn/model.py).

Run from the repository root:  python tests/golden/make_gdn_golden.py
The reference ships no GDN vector, so this fixture pins the oracle against
itself over time (a later edit of the oracle that changes its results fails the
CPU test) and gives the GPU test a file-based expectation that does not depend on
running the oracle. Stored: the seed, the full output o [4,8,128] and every 61st
element of the flattened new state (61 is coprime to 128, so the sample walks
across rows and columns).
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "tests"))
from conftest import load_oracle  # noqa: E402

STRIDE = 61


def main():
    torch.set_num_threads(1)
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 0})
    m.reseed()
    inputs = m.get_inputs()
    with torch.no_grad():
        o, s_new = m.Model(*m.get_init_inputs())(*inputs)
    out = Path(__file__).with_name("gdn_config0.npz")
    np.savez_compressed(out, seed=np.int64(1234), stride=np.int64(STRIDE), o=o.numpy(),
                        state_sample=s_new.flatten()[::STRIDE].numpy())
    print("wrote", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
