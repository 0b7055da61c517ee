"""A decode loop as one CUDA graph.

The GDN decode step is a single kernel over pre-allocated buffers, so a run of steps whose inputs
are already on the device (a multi-step serving loop, or the 64 pre-generated steps of the bench
workload) can be recorded once and replayed with one launch call per run instead of one per step.
Nothing is computed in torch: the graph holds the launches that ``capi.gdn_decode`` makes.
"""
from __future__ import annotations

import torch

from . import capi


class GdnDecodeGraph:
    """Records ``len(q)`` decode steps on ``state`` (updated in place) and replays them.

    ``q, k, v, g, beta`` are stacks of per-step inputs ``[steps, ...]``; ``out`` is ``[steps, B, Hv, 128]``
    (one output slice per step) or ``[B, Hv, 128]`` (every step overwrites it). The tensors must stay
    alive and at the same addresses for as long as the graph is replayed; new inputs are copied into
    them between replays.
    """

    def __init__(self, state, out, q, k, v, g, beta, config: int = 0, zigzag: bool = True):
        self.tensors = (state, out, q, k, v, g, beta)
        steps = q.shape[0]
        per_step_out = out.dim() == 4
        capi.lib()
        # one eager step first: nothing inside the capture may be a first-time initialisation
        warm = state.clone()
        capi.gdn_decode(warm, out[0] if per_step_out else out, q[0], k[0], v[0], g[0], beta[0], config)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            for s in range(steps):
                # zig-zag: odd steps walk the state backwards, so each starts on what its predecessor left in L2
                cfg = capi.gdn_loop_config(s, config) if zigzag else config
                capi.gdn_decode(state, out[s] if per_step_out else out, q[s], k[s], v[s], g[s], beta[s], cfg)
        self.steps = steps

    def replay(self) -> None:
        self.graph.replay()
