"""Device-side set-up, timed steps and CPU-baseline samples for the workloads of ``bench.py``.

Nothing here computes an operator's result in torch on the timed GPU path: torch draws the synthetic
inputs (and quantises the synthetic weights once, untimed); every timed GPU step is a call into the C ABI
or into ``cuda_extension``. The ``cpu_*`` functions time the eager oracles on the host cores (the reported
CPU baseline), and ``MoeEpWorkload.parity`` is the checker leg of the expert-parallel line.
"""
from __future__ import annotations

import importlib.util
import os
import time
from pathlib import Path

import torch

from cuda_agent_b200 import capi, load_extension

ROOT = Path(__file__).resolve().parent
FP8_MAX = 448.0


def load_oracle(name: str, env: dict | None = None):
    """oracle/<name>/model.py as a module (test infrastructure: CPU baseline and checker legs only)."""
    for key, val in (env or {}).items():
        os.environ[key] = str(val)
    spec = importlib.util.spec_from_file_location(f"{name}_oracle_bench", ROOT / "oracle" / name / "model.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def quant_128x128(w: torch.Tensor):
    """Untimed set-up: 128x128 block quantisation of synthetic weights on the device."""
    *lead, N, K = w.shape
    blocks = w.reshape(*lead, N // 128, 128, K // 128, 128)
    scale = blocks.abs().amax(dim=(-3, -1)).clamp_min(1e-4) / FP8_MAX
    q = (blocks / scale[..., :, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(*lead, N, K), scale.contiguous()


def expert_weights(dev, seed: int, expert: int, H: int, I: int):
    """The synthetic weights of one expert, N(0, 0.02) quantised 128x128: a function of (seed, expert id)
    alone, so that any rank can draw any expert's weights again (the parity leg does)."""
    gen = torch.Generator(device=dev).manual_seed(seed * 100003 + expert)
    w13 = quant_128x128(torch.randn(2 * I, H, device=dev, generator=gen) * 0.02)
    w2 = quant_128x128(torch.randn(H, I, device=dev, generator=gen) * 0.02)
    return w13[0], w13[1], w2[0], w2[1]


# --------------------------------------------------------------------------------------------- GDN
class GdnWorkload:
    """Gated DeltaNet decode at serving scale: B=256 sequences, 16 q/k heads shared by groups of 2 across 32
    value heads, dk=dv=128, fp32 state of 512 MiB; 64 distinct seeded decode steps taken in turn."""
    D, B, HQ, HV, N_DISTINCT = 128, 256, 16, 32, 64

    def __init__(self, dev, seed):
        D, B, HQ, HV, n = self.D, self.B, self.HQ, self.HV, self.N_DISTINCT
        gen = torch.Generator(device=dev).manual_seed(seed)
        q = torch.randn(n, B, HQ, D, device=dev, generator=gen)
        self.q = (q / q.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
        k = torch.randn(n, B, HQ, D, device=dev, generator=gen)
        self.k = (k / k.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
        self.v = torch.randn(n, B, HV, D, device=dev, generator=gen).to(torch.bfloat16)
        self.g = -torch.nn.functional.softplus(torch.randn(n, B, HV, device=dev, generator=gen))
        self.beta = torch.sigmoid(torch.randn(n, B, HV, device=dev, generator=gen))
        self.state = torch.randn(B, HV, D, D, device=dev, generator=gen) * 0.02
        self.out = torch.empty(B, HV, D, device=dev)
        self.dev = dev
        self.bytes_per_step = 2 * B * HV * D * D * 4 + 2 * B * HQ * D * 2 + B * HV * D * 2 + 2 * B * HV * 4 + B * HV * D * 4
        self.h2d_bytes = 2 * B * HQ * D * 2 + B * HV * D * 2 + 2 * B * HV * 4
        self.d2h_bytes = B * HV * D * 4

    def step(self, i, config=0, zigzag=True):
        j = i % self.N_DISTINCT
        cfg = capi.gdn_loop_config(i, config) if zigzag else config
        capi.gdn_decode(self.state, self.out, self.q[j], self.k[j], self.v[j], self.g[j], self.beta[j], cfg)

    def make_e2e(self, config=0, zigzag=True):
        """End-to-end step through cuda_extension.gdn_decode_forward. A step's q/k/v/g/beta sit in ONE pinned
        staging record and reach the GPU with one copy; the output goes back with one copy; uploads, compute
        and downloads of neighbouring steps overlap on three streams (two slots)."""
        ext = load_extension()
        B, HQ, HV, D, n = self.B, self.HQ, self.HV, self.D, self.N_DISTINCT
        sizes = [B * HQ * D * 2, B * HQ * D * 2, B * HV * D * 2, B * HV * 4, B * HV * 4]
        offs = [sum(sizes[:i]) for i in range(6)]
        host = torch.empty(n, offs[5], dtype=torch.uint8).pin_memory()
        for j in range(n):
            for part, t in enumerate((self.q[j], self.k[j], self.v[j], self.g[j], self.beta[j])):
                host[j, offs[part]:offs[part + 1]] = t.contiguous().view(torch.uint8).reshape(-1).cpu()
        slots = [torch.empty(offs[5], dtype=torch.uint8, device=self.dev) for _ in range(2)]

        def views(buf):
            return (buf[offs[0]:offs[1]].view(torch.bfloat16).view(B, HQ, D),
                    buf[offs[1]:offs[2]].view(torch.bfloat16).view(B, HQ, D),
                    buf[offs[2]:offs[3]].view(torch.bfloat16).view(B, HV, D),
                    buf[offs[3]:offs[4]].view(torch.float32).view(B, HV),
                    buf[offs[4]:offs[5]].view(torch.float32).view(B, HV))
        slot_views = [views(b) for b in slots]
        host_out = torch.empty(2, B, HV, D).pin_memory()
        state = self.state

        def upload(i, s):
            slots[s].copy_(host[i % n], non_blocking=True)

        def compute(i, s):
            o, _ = ext.gdn_decode_forward(state, *slot_views[s], capi.gdn_loop_config(i, config) if zigzag else config)
            return o

        def download(o, s):
            host_out[s].copy_(o, non_blocking=True)
        return Pipeline(self.dev, upload, compute, download)


class Pipeline:
    """Two-slot software pipeline over three CUDA streams: the host->device copy of step i+1 and the
    device->host copy of step i-1 run beside the kernels of step i. run(n) enqueues n steps and waits."""

    def __init__(self, dev, upload, compute, download):
        self.dev, self.upload, self.compute, self.download = dev, upload, compute, download
        self.copy_in, self.copy_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.in_ready = [torch.cuda.Event() for _ in range(2)]
        self.in_free = [torch.cuda.Event() for _ in range(2)]

    def run(self, n):
        stream = torch.cuda.current_stream(self.dev)
        for e in self.in_free:
            e.record(stream)

        def up(i):
            s = i % 2
            with torch.cuda.stream(self.copy_in):
                self.copy_in.wait_event(self.in_free[s])
                self.upload(i, s)
                self.in_ready[s].record(self.copy_in)
        up(0)
        for i in range(n):
            s = i % 2
            if i + 1 < n:
                up(i + 1)
            stream.wait_event(self.in_ready[s])
            out = self.compute(i, s)
            self.in_free[s].record(stream)
            done = torch.cuda.Event()
            done.record(stream)
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(done)
                self.download(out, s)
                out.record_stream(self.copy_out)
        self.copy_out.synchronize()
        stream.synchronize()


# --------------------------------------------------------------------------------------------- MoE, one GPU
class MoeWorkload:
    """FP8 MoE layer, one GPU: T tokens, hidden H, intermediate I, E experts, top-k softmax routing."""

    def __init__(self, dev, T=4096, H=2048, I=1024, E=64, k=6, seed=1237):
        self.T, self.H, self.I, self.E, self.k, self.dev = T, H, I, E, k, dev
        gen = torch.Generator(device=dev).manual_seed(seed)
        self.x = torch.randn(T, H, device=dev, generator=gen).to(torch.bfloat16)
        self.router_w = (torch.randn(E, H, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        self.router_bias = torch.zeros(E, device=dev)
        ws = [expert_weights(dev, seed, e, H, I) for e in range(E)]
        self.w13_q = torch.stack([w[0] for w in ws]); self.w13_s = torch.stack([w[1] for w in ws])
        self.w2_q = torch.stack([w[2] for w in ws]); self.w2_s = torch.stack([w[3] for w in ws])
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

    def make_e2e(self, config=0):
        hx = self.x.cpu().pin_memory()
        ho = torch.empty(2, *self.x.shape, dtype=torch.bfloat16).pin_memory()
        dx = [torch.empty_like(self.x) for _ in range(2)]
        self.h2d_bytes, self.d2h_bytes = hx.numel() * 2, hx.numel() * 2
        return Pipeline(self.dev, lambda i, s: dx[s].copy_(hx, non_blocking=True),
                        lambda i, s: self.layer_step(dx[s], config),
                        lambda o, s: ho[s].copy_(o, non_blocking=True))


# --------------------------------------------------------------------------------------------- MoE, expert parallel
class MoeEpWorkload:
    """DeepSeek-V3-shaped expert-parallel layer: T tokens per GPU, H 7168, I 2048, 256 routed experts in
    blocks of 256/N per rank, top-8 sigmoid routing with 8 groups / top-4, one shared expert."""
    SHARED_ID = 100000      # expert id under which the shared expert's weights are drawn

    def __init__(self, dev, rank, world, T=8192, H=7168, I=2048, E=256, k=8, seed=1238, mode="peer", group=None,
                 gemm_ctas=0, connect=True):
        from cuda_agent_b200 import ep
        self.T, self.H, self.I, self.E, self.k, self.world, self.rank = T, H, I, E, k, world, rank
        self.dev, self.seed, self.mode = dev, seed, mode
        gen = torch.Generator(device=dev).manual_seed(seed)           # same router on every rank
        self.router_w = (torch.randn(E, H, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        self.router_bias = torch.randn(E, device=dev, generator=gen) * 0.02
        gen_r = torch.Generator(device=dev).manual_seed(seed + 1 + rank)
        self.x = torch.randn(T, H, device=dev, generator=gen_r).to(torch.bfloat16)
        el = E // world
        w13_q = torch.empty(el, 2 * I, H, dtype=torch.float8_e4m3fn, device=dev)
        w13_s = torch.empty(el, 2 * I // 128, H // 128, device=dev)
        w2_q = torch.empty(el, H, I, dtype=torch.float8_e4m3fn, device=dev)
        w2_s = torch.empty(el, H // 128, I // 128, device=dev)
        for e in range(el):
            w13_q[e], w13_s[e], w2_q[e], w2_s[e] = expert_weights(dev, seed, rank * el + e, H, I)
        shared = expert_weights(dev, seed, self.SHARED_ID, H, I)
        self.ops = ep.CudaOps(self.router_w, self.router_bias, w13_q, w13_s, w2_q, w2_s, shared, k=k,
                              routing=1, n_group=8, topk_group=4, scaling=1.0, num_experts=E, gemm_ctas=gemm_ctas)
        # connect=False: the caller joins several ranks of one process itself (PeerLayer.build_local)
        self.layer = ep.make_layer(self.ops, rank, world, T, mode=mode, group=group) if connect else None
        self.flops_per_gpu = 6 * T * k * H * I + 6 * T * H * I          # routed + shared expert GEMMs

    def step(self, x=None):
        return self.layer.forward(self.x if x is None else x)

    def make_e2e(self):
        hx = self.x.cpu().pin_memory()
        ho = torch.empty(2, *self.x.shape, dtype=torch.bfloat16).pin_memory()
        dx = [torch.empty_like(self.x) for _ in range(2)]
        self.h2d_bytes, self.d2h_bytes = hx.numel() * 2, hx.numel() * 2
        return Pipeline(self.dev, lambda i, s: dx[s].copy_(hx, non_blocking=True),
                        lambda i, s: self.step(dx[s]),
                        lambda o, s: ho[s].copy_(o, non_blocking=True))

    def parity(self, out, n_tokens=256):
        """Checker leg (outside every timed region): `out` on the first n_tokens local tokens against the eager
        oracle's own functions run on this GPU, with every touched expert's weights drawn again. Returns
        rel_l2 over all those tokens, the number of tokens whose expert set differs from the oracle's (its
        logits are cuBLAS sums in another order, so a near-tie may fall the other way) and rel_l2 over the
        tokens routed identically."""
        m = load_oracle("moe", {"CAB_MOE_CONFIG": 4})
        x = self.x[:n_tokens]
        with torch.no_grad():
            logits = x.float() @ self.router_w.float().t()
            idx, w = m.route_sigmoid_group_topk(logits, self.router_bias, self.k, 8, 4, 1.0)
            got_idx, _ = self.ops.route(x.contiguous())
            same = (got_idx == idx).all(dim=1)
            xq, sx = m.quant_1x128(x.float())
            # every entry's FFN output rounded to bf16, then the weighted sum in ascending slot order, as the
            # oracle's Model.forward forms it
            y_slots = torch.zeros(n_tokens, self.k, self.H, dtype=torch.bfloat16, device=self.dev)
            for e in torch.unique(idx).tolist():
                tok, slot = torch.nonzero(idx == e, as_tuple=True)
                w13_q, w13_s, w2_q, w2_s = expert_weights(self.dev, self.seed, e, self.H, self.I)
                y_slots[tok, slot] = m.expert_ffn(xq[tok], sx[tok], w13_q, w13_s, w2_q, w2_s).to(torch.bfloat16)
            ref = torch.zeros(n_tokens, self.H, device=self.dev)
            for s in range(self.k):
                ref = ref + w[:, s, None] * y_slots[:, s].float()
            sh = expert_weights(self.dev, self.seed, self.SHARED_ID, self.H, self.I)
            ref = ref + m.expert_ffn(xq, sx, *sh).to(torch.bfloat16).float()
            ref = ref.to(torch.bfloat16).float()
        got = out[:n_tokens].float()
        rel = lambda a, b: float((a - b).norm() / b.norm())
        return {"rel_l2": round(rel(got, ref), 5), "tokens": n_tokens,
                "tokens_routed_differently": int((~same).sum()),
                "rel_l2_identically_routed": round(rel(got[same], ref[same]), 5)}


# --------------------------------------------------------------------------------------------- sparse MLA
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
        lens = self.seq_len.cpu().tolist()
        for b in range(B):
            chosen = torch.randperm(lens[b], device=dev, generator=gen)[:topk].to(torch.int32)
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

    def make_e2e(self, nsplit=0, config=0):
        """q / idx / seq_len of a step in one pinned staging record (one copy up), the output back with one
        copy; the cache is resident, as in serving."""
        sizes = [self.q.numel() * 2, self.idx.numel() * 4, self.seq_len.numel() * 4]
        offs = [0, sizes[0], sizes[0] + sizes[1], sum(sizes)]
        host = torch.empty(offs[3], dtype=torch.uint8).pin_memory()
        for part, t in enumerate((self.q, self.idx, self.seq_len)):
            host[offs[part]:offs[part + 1]] = t.contiguous().view(torch.uint8).reshape(-1).cpu()
        slots = [torch.empty(offs[3], dtype=torch.uint8, device=self.dev) for _ in range(2)]
        views = [(b[offs[0]:offs[1]].view(torch.bfloat16).view_as(self.q),
                  b[offs[1]:offs[2]].view(torch.int32).view_as(self.idx),
                  b[offs[2]:offs[3]].view(torch.int32).view_as(self.seq_len)) for b in slots]
        ho = torch.empty(2, *self.out.shape, dtype=torch.bfloat16).pin_memory()
        self.h2d_bytes, self.d2h_bytes = offs[3], self.out.numel() * 2
        ext, kv, scale = self.ext, self.kv, self.scale
        return Pipeline(self.dev, lambda i, s: slots[s].copy_(host, non_blocking=True),
                        lambda i, s: ext.mla_sparse_decode_forward(views[s][0], kv, views[s][2], views[s][1], scale,
                                                                   nsplit, False, config),
                        lambda o, s: ho[s].copy_(o, non_blocking=True))


# --------------------------------------------------------------------------------------------- yardstick
def library_fp8_gemm_tflops(dev, n=8192, burst_iters=10, sustained_s=0.5):
    """What the vendor library's dense e4m3 GEMM (torch._scaled_mm -> cuBLASLt, per-tensor scales, n^3) reaches on
    this GPU right now: (best single call, average over `sustained_s` of back-to-back calls), TFLOP/s. A yardstick
    for the roofline record only (no measured fp8 peak is provided); nothing of the product calls it."""
    a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()          # column-major second operand
    one = torch.ones((), device=dev)
    run = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    best = 0.0
    for _ in range(burst_iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); run(); e1.record()
        torch.cuda.synchronize()
        best = max(best, 2.0 * n ** 3 / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    iters = max(10, int(sustained_s / (2.0 * n ** 3 / (best * 1e12))))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    return best, 2.0 * n ** 3 * iters / (e0.elapsed_time(e1) * 1e-3) / 1e12


# --------------------------------------------------------------------------------------------- timing helpers
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


# --------------------------------------------------------------------------------------------- CPU baselines
def cpu_threads() -> int:
    """Use every host core: a launcher such as torchrun exports OMP_NUM_THREADS=1 to its children."""
    n = os.cpu_count() or 1
    if torch.get_num_threads() != n:
        torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_gdn(budget_s: float, n_steps: int = 20, n_warmup: int = 1):
    """Eager GDN oracle on the host cores: (GB/s, s per step, sample text, threads)."""
    wl = GdnWorkload
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 1})
    threads = cpu_threads()
    gen = torch.Generator().manual_seed(1235)
    model = m.Model(8, wl.HQ, wl.HV)
    S = m.make_state(8, wl.HV, gen)
    step = m.make_step_inputs(8, wl.HQ, wl.HV, gen)
    with torch.no_grad():
        model(S, *step)
        t0 = time.perf_counter()
        model(S, *step)
        per_row = (time.perf_counter() - t0) / 8
    total = max(1, n_steps + n_warmup)
    b_sample = int(min(wl.B, max(8, budget_s / (per_row * total))))
    b_sample -= b_sample % 8
    model = m.Model(b_sample, wl.HQ, wl.HV)
    S = m.make_state(b_sample, wl.HV, gen)
    steps = [m.make_step_inputs(b_sample, wl.HQ, wl.HV, gen) for _ in range(min(4, total))]
    with torch.no_grad():
        for i in range(n_warmup):
            _, S = model(S, *steps[i % len(steps)])
        t0 = time.perf_counter()
        for i in range(n_steps):
            _, S = model(S, *steps[i % len(steps)])
        dt = (time.perf_counter() - t0) / max(1, n_steps)
    D, B, HQ, HV = wl.D, wl.B, wl.HQ, wl.HV
    bytes_per_step = 2 * B * HV * D * D * 4 + 2 * B * HQ * D * 2 + B * HV * D * 2 + 2 * B * HV * 4 + B * HV * D * 4
    gbs = bytes_per_step * (b_sample / B) / dt / 1e9
    return gbs, dt, f"{n_steps} steps of {b_sample} of the {B} batch rows (all 32 value heads), torch eager fp32", threads


def cpu_moe(repeats: int = 1):
    """Eager MoE oracle (config 3, full size) on the host cores: (TFLOP/s of the grouped-GEMM FLOP, s per
    layer call, sample text, threads). Weights are drawn by the oracle itself on the CPU, untimed."""
    threads = cpu_threads()
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 3})
    m.reseed()
    model = m.Model(*m.get_init_inputs())
    (x,) = m.get_inputs()
    with torch.no_grad():
        t0 = time.perf_counter()
        for _ in range(repeats):
            model(x)
        dt = (time.perf_counter() - t0) / repeats
    flops = 6 * model.T * model.k * model.H * model.I
    return flops / dt / 1e12, dt, f"{repeats} full layer call(s): 4096 tokens, 64 experts, top-6, torch eager fp32 on dequantised operands", threads


def cpu_mla(wl: "MlaWorkload", n_seq: int = 16):
    """Eager MLA oracle on the host cores over the first n_seq sequences of the GPU workload's own inputs
    (attention only: the cache is copied from the GPU, untimed): (tok/s, s per sequence, sample, threads)."""
    threads = cpu_threads()
    m = load_oracle("mla", {"CAB_MLA_CONFIG": 2})
    q, kv = wl.q[:n_seq].cpu(), wl.kv[:n_seq].cpu()
    seq_len, idx = wl.seq_len[:n_seq].cpu(), wl.idx[:n_seq].cpu()
    model = m.Model(n_seq, wl.Hh, wl.S, wl.topk)
    with torch.no_grad():
        model(q[:2], kv[:2], seq_len[:2], idx[:2])
        t0 = time.perf_counter()
        model(q, kv, seq_len, idx)
        dt = time.perf_counter() - t0
    return n_seq / dt, dt / n_seq, f"{n_seq} of the 64 sequences (128 heads, 2048 selected rows each), torch eager fp32", threads


def cpu_moe_ep(n_experts: int = 6, rows_per_expert: int = 256, H: int = 7168, I: int = 2048):
    """Expert FFN of the expert-parallel layer on the host cores for a subset of experts with the row count a
    balanced layer gives each (8192 * 8 / 256 = 256): (TFLOP/s, seconds, sample text, threads). The layer's
    figure is a linear extrapolation: every expert costs the same."""
    threads = cpu_threads()
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 4})
    gen = torch.Generator().manual_seed(77)
    xq, sx = m.quant_1x128(torch.randn(rows_per_expert, H, generator=gen))
    experts = []
    for _ in range(2):                                   # two distinct weight sets, reused in turn (untimed set-up)
        experts.append(m.quant_128x128(torch.randn(2 * I, H, generator=gen) * 0.02)
                       + m.quant_128x128(torch.randn(H, I, generator=gen) * 0.02))
    with torch.no_grad():
        m.expert_ffn(xq, sx, *experts[0])
        t0 = time.perf_counter()
        for e in range(n_experts):
            m.expert_ffn(xq, sx, *experts[e % 2])
        dt = time.perf_counter() - t0
    flops = 6 * rows_per_expert * H * I * n_experts
    return flops / dt / 1e12, dt, (f"{n_experts} of 256 experts x {rows_per_expert} rows (the balanced share of 8192 tokens, "
                                   f"top-8), torch eager fp32 on dequantised operands; per-layer figure = linear extrapolation"), threads
