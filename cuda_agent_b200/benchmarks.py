"""Device-side set-up and timed steps for the MoE and MLA workloads of ``bench.py``.

Nothing here computes an operator's result in torch: torch is used to draw the
synthetic inputs (and to quantise the synthetic weights once, untimed); every
timed step is a call into the C ABI or into ``cuda_extension``.
"""
from __future__ import annotations

import torch

from . import capi, load_extension

FP8_MAX = 448.0


def quant_128x128(w: torch.Tensor):
    """Untimed set-up: 128x128 block quantisation of synthetic weights on the device."""
    *lead, N, K = w.shape
    blocks = w.reshape(*lead, N // 128, 128, K // 128, 128)
    scale = blocks.abs().amax(dim=(-3, -1)).clamp_min(1e-4) / FP8_MAX
    q = (blocks / scale[..., :, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(*lead, N, K), scale.contiguous()


class MoeWorkload:
    """FP8 MoE layer, one GPU: T tokens, hidden H, intermediate I, E experts, top-k softmax routing."""

    def __init__(self, dev, T=4096, H=2048, I=1024, E=64, k=6, seed=1237):
        self.T, self.H, self.I, self.E, self.k, self.dev = T, H, I, E, k, dev
        gen = torch.Generator(device=dev).manual_seed(seed)
        self.x = torch.randn(T, H, device=dev, generator=gen).to(torch.bfloat16)
        self.router_w = (torch.randn(E, H, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        self.router_bias = torch.zeros(E, device=dev)
        w13, w2 = [], []
        for _ in range(E):
            w13.append(quant_128x128(torch.randn(2 * I, H, device=dev, generator=gen) * 0.02))
            w2.append(quant_128x128(torch.randn(H, I, device=dev, generator=gen) * 0.02))
        self.w13_q = torch.stack([q for q, _ in w13]); self.w13_s = torch.stack([s for _, s in w13])
        self.w2_q = torch.stack([q for q, _ in w2]); self.w2_s = torch.stack([s for _, s in w2])
        self.ext = load_extension()
        # intermediates for timing the two GEMMs on their own
        idx, self.w = self.ext.moe_route(self.x, self.router_w, self.router_bias, k, 0, 1, 1, 1.0)
        self.perm = capi.moe_permute(idx, E)
        cap = self.perm["max_tiles"] * 128
        self.a_q = torch.empty(cap, H, dtype=torch.uint8, device=dev)
        self.a_s = torch.empty(H // 128, cap, device=dev)
        capi.moe_quant_dispatch(self.a_q, self.a_s, self.x, self.perm["dst_row"], k)
        self.h_q = torch.empty(cap, I, dtype=torch.uint8, device=dev)
        self.h_s = torch.empty(I // 128, cap, device=dev)
        self.y = torch.empty(cap, H, dtype=torch.bfloat16, device=dev)
        self.status = torch.zeros(2, dtype=torch.int32, device=dev)
        self.gemm_flops = 6 * T * k * H * I
        self.min_bytes = self.w13_q.numel() + self.w2_q.numel() + 4 * (self.w13_s.numel() + self.w2_s.numel()) \
            + 2 * self.x.numel() * 2

    def gemm_step(self, config=0):
        p = self.perm
        capi.moe_grouped_gemm_fp8(0, self.h_q, self.h_s, self.a_q, self.a_s, self.w13_q.view(torch.uint8), self.w13_s,
                                  p["tile_expert"], p["num_tiles"], p["max_tiles"], self.status[0:1], config)
        capi.moe_grouped_gemm_fp8(1, self.y, None, self.h_q, self.h_s, self.w2_q.view(torch.uint8), self.w2_s,
                                  p["tile_expert"], p["num_tiles"], p["max_tiles"], self.status[1:2], config)

    def layer_step(self, x=None, config=0):
        return self.ext.moe_forward(self.x if x is None else x, self.router_w, self.router_bias, self.w13_q,
                                    self.w13_s, self.w2_q, self.w2_s, None, None, None, None, self.k, 0, 1, 1, 1.0,
                                    False, config)


class MoeEpWorkload:
    """DeepSeek-V3-shaped expert-parallel layer: T tokens per GPU, H 7168, I 2048, 256 routed experts in
    blocks of 256/N per rank, top-8 sigmoid routing with 8 groups / top-4, one shared expert."""

    def __init__(self, dev, rank, world, T=8192, H=7168, I=2048, E=256, k=8, seed=1238, micro_batches=None, dedup=None,
                 gemm_ctas=0):
        from .ep import CudaOps
        self.T, self.H, self.I, self.E, self.k, self.world = T, H, I, E, k, world
        gen = torch.Generator(device=dev).manual_seed(seed)           # same router on every rank
        router_w = (torch.randn(E, H, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        router_bias = torch.randn(E, device=dev, generator=gen) * 0.02
        gen_r = torch.Generator(device=dev).manual_seed(seed + 1 + rank)
        self.x = torch.randn(T, H, device=dev, generator=gen_r).to(torch.bfloat16)
        el = E // world
        w13_q = torch.empty(el, 2 * I, H, dtype=torch.float8_e4m3fn, device=dev)
        w13_s = torch.empty(el, 2 * I // 128, H // 128, device=dev)
        w2_q = torch.empty(el, H, I, dtype=torch.float8_e4m3fn, device=dev)
        w2_s = torch.empty(el, H // 128, I // 128, device=dev)
        for e in range(el):
            w13_q[e], w13_s[e] = quant_128x128(torch.randn(2 * I, H, device=dev, generator=gen_r) * 0.02)
            w2_q[e], w2_s[e] = quant_128x128(torch.randn(H, I, device=dev, generator=gen_r) * 0.02)
        s13 = quant_128x128(torch.randn(2 * I, H, device=dev, generator=gen_r) * 0.02)
        s2 = quant_128x128(torch.randn(H, I, device=dev, generator=gen_r) * 0.02)
        self.ops = CudaOps(router_w, router_bias, w13_q, w13_s, w2_q, w2_s, (s13[0], s13[1], s2[0], s2[1]), k=k,
                           routing=1, n_group=8, topk_group=4, scaling=1.0, num_experts=E, gemm_ctas=gemm_ctas)
        self.micro_batches = micro_batches if micro_batches is not None else 1
        self.dedup = dedup
        self.flops_per_gpu = 6 * T * k * H * I + 6 * T * H * I          # routed + shared expert GEMMs

    def step(self, x=None):
        from .ep import ep_moe_forward
        return ep_moe_forward(self.x if x is None else x, self.ops, self.world,
                              micro_batches=self.micro_batches, dedup=self.dedup)


class MlaWorkload:
    """Top-k sparse MLA decode: B sequences, 128 heads, 2048 of up to 32768 cached rows each."""

    def __init__(self, dev, B=64, Hh=128, S=32768, topk=2048, min_len=8192, seed=1236):
        self.B, self.Hh, self.S, self.topk, self.dev = B, Hh, S, topk, dev
        gen = torch.Generator(device=dev).manual_seed(seed)
        self.q = torch.randn(B, 1, Hh, 576, device=dev, generator=gen).to(torch.bfloat16)
        self.kv = torch.empty(B, S, 576, dtype=torch.bfloat16, device=dev)
        for b in range(B):
            self.kv[b] = torch.randn(S, 576, device=dev, generator=gen).to(torch.bfloat16)
        self.seq_len = torch.randint(min_len, S + 1, (B,), device=dev, generator=gen, dtype=torch.int32)
        idx = torch.full((B, 1, topk), -1, dtype=torch.int32, device=dev)
        for b in range(B):
            n = int(self.seq_len[b])
            chosen = torch.randperm(n, device=dev, generator=gen)[:topk].to(torch.int32)
            idx[b, 0, : chosen.numel()] = chosen
        self.idx = idx
        self.out = torch.empty(B, 1, Hh, 512, dtype=torch.bfloat16, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.scale = 192 ** -0.5
        self.ext = load_extension()
        self.bytes = B * topk * 576 * 2 + self.q.numel() * 2 + self.out.numel() * 2 + idx.numel() * 4
        self.flops = 2 * B * Hh * topk * (576 + 512)
        self.scratch = {}

    def step(self, nsplit=1, config=0):
        if nsplit not in self.scratch:
            n = capi.mla_scratch_bytes(self.B, self.Hh, nsplit)
            self.scratch[nsplit] = torch.empty(max(n, 16), dtype=torch.uint8, device=self.dev) if n else None
        capi.mla_sparse_decode(self.out, self.q, self.kv, self.seq_len, self.idx, self.scale, nsplit,
                               self.scratch[nsplit], self.status, config)

    def api_step(self, q, idx, seq_len):
        return self.ext.mla_sparse_decode_forward(q, self.kv, seq_len, idx, self.scale, 0, False, 0)


def time_cuda(fn, steps: int, warmup: int) -> float:
    """Milliseconds per call between two CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps
