#!/usr/bin/env python3
"""Headline benchmark: Gated DeltaNet decode at serving scale, in GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload ("gdn_decode_serving"): B=256 sequences per GPU, 16 q/k heads shared by
groups of 2 across 32 value heads, dk=dv=128, fp32 state of 512 MiB per GPU. One
step is one decode step (one kernel launch over the whole batch) with that
step's own q/k/v/g/beta, taken in turn from 64 pre-generated seeded steps.
Algorithmic bytes per step per GPU: state read + write 2*536870912, q and k
2*1048576, v 2097152, g and beta 2*32768, o 4194304 = 1082195968.

Printed keys (one JSON line, rank 0):
  value      GB/s over all GPUs with every input already in HBM (CUDA events, max over ranks)
  e2e        same metric through cuda_extension.gdn_decode_forward with the step's
             q/k/v/g/beta coming from pinned host memory and o going back to it,
             copies inside the timed region (the 512 MiB state lives on the GPU
             between steps, as it does in a serving process)
  roofline   the decode kernel against measured HBM copy bandwidth
  cpu_baseline  the eager oracle on this box's host cores (a reported baseline)
  clocks     SM clock and throttle reasons sampled during the timed regions

With N > 1 the batch is sharded with no collective: every rank runs the same
per-GPU workload on its own state (weak scaling); NCCL is used only for the
barrier and the max over ranks.

``--impl reference`` times the eager CPU oracle (the reference's torch-eager path
for this operator) on the host cores instead; rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

D = 128
B, HQ, HV = 256, 16, 32
N_DISTINCT_STEPS = 64
BYTES_PER_STEP = 2 * B * HV * D * D * 4 + 2 * B * HQ * D * 2 + B * HV * D * 2 + 2 * B * HV * 4 + B * HV * D * 4
H2D_BYTES = 2 * B * HQ * D * 2 + B * HV * D * 2 + 2 * B * HV * 4
D2H_BYTES = B * HV * D * 4
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one gdn_decode_kernel launch at this
# workload, from the ncu capture summarised in profiles/gdn_decode_kernel_config1.md.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 1025223168


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=640)
    ap.add_argument("--warmup", type=int, default=64)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--config", type=int, default=0, help="launcher variant passed to the op")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-dedup", action="store_true",
                    help="moe_ep: send one row per (token, expert) instead of one per (token, destination rank)")
    ap.add_argument("--graph", action="store_true",
                    help="gdn: also time the loop recorded as CUDA graphs (extra key \"cuda_graph\")")
    ap.add_argument("--workload", choices=["gdn", "moe", "mla", "moe_ep"], default="gdn",
                    help="gdn = the headline line; moe = FP8 MoE layer (4096 tokens, 64 experts, top-6); "
                         "mla = top-2048 sparse MLA decode (64 sequences, 128 heads)")
    ap.add_argument("--micro-batches", type=int, default=1,
                    help="moe_ep: token micro-batches pipelined over streams (with --config C < 148 GEMM CTAs)")
    ap.add_argument("--nsplit", type=int, default=1, help="mla: splits of the selected rows per CTA group")
    return ap.parse_args()


# --------------------------------------------------------------------------- clocks
REASON_BITS = {
    0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
    0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
}


class ClockSampler:
    """Reads SM clock and clock-event reasons through NVML every few ms (read-only)."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.samples = []  # (monotonic time, sm_mhz, reasons bitmask)
        self.period = period_s
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            if visible:
                token = visible.split(",")[index]
                index = int(token) if token.isdigit() else index
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _loop(self):
        nv = self._nvml
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                self.samples.append((time.monotonic(), mhz, int(get_reasons(self._h))))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self, windows):
        """Median SM MHz and union of reasons over samples inside the [t0, t1] windows."""
        inside = [s for s in self.samples if any(a <= s[0] <= b for a, b in windows)]
        scope = "timed regions"
        if len(inside) < 3:
            inside, scope = self.samples, "whole run (timed regions shorter than the sampling period)"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0,
                    "note": "NVML unavailable"}
        mhz = sorted(s[1] for s in inside)
        mask = 0
        for s in inside:
            mask |= s[2]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": sorted(name for bit, name in REASON_BITS.items() if mask & bit),
                "samples": len(inside), "scope": scope}


# --------------------------------------------------------------------------- reference arm
def load_oracle():
    import importlib.util
    os.environ["CAB_GDN_CONFIG"] = "1"
    spec = importlib.util.spec_from_file_location("gdn_oracle_model", ROOT / "oracle" / "gdn" / "model.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def time_oracle_cpu(n_steps: int, n_warmup: int, budget_s: float):
    """Eager oracle on the host cores. Returns (GB/s, seconds per step, sample text, threads)."""
    import torch
    m = load_oracle()
    threads = torch.get_num_threads()
    gen = torch.Generator().manual_seed(1235)
    # calibrate on 8 batch rows, then pick the batch sample that fits the budget
    model = m.Model(8, HQ, HV)
    S = m.make_state(8, HV, gen)
    step = m.make_step_inputs(8, HQ, HV, gen)
    with torch.no_grad():
        model(S, *step)
        t0 = time.perf_counter()
        model(S, *step)
        per_row = (time.perf_counter() - t0) / 8
    total_steps = max(1, n_steps + n_warmup)
    b_sample = int(min(B, max(8, budget_s / (per_row * total_steps))))
    b_sample -= b_sample % 8
    model = m.Model(b_sample, HQ, HV)
    S = m.make_state(b_sample, HV, gen)
    steps = [m.make_step_inputs(b_sample, HQ, HV, gen) for _ in range(min(4, total_steps))]
    with torch.no_grad():
        for i in range(n_warmup):
            _, S = model(S, *steps[i % len(steps)])
        t0 = time.perf_counter()
        for i in range(n_steps):
            _, S = model(S, *steps[i % len(steps)])
        dt = (time.perf_counter() - t0) / max(1, n_steps)
    gbs = BYTES_PER_STEP * (b_sample / B) / dt / 1e9
    sample = f"{n_steps} steps of {b_sample} of the {B} batch rows (all 32 value heads), torch eager fp32"
    return gbs, dt, sample, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    gbs, dt, sample, threads = time_oracle_cpu(args.steps, args.warmup, budget_s=150.0)
    line = {
        "impl": "reference", "metric": "gdn_decode_gbps", "value": round(gbs, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": "gdn_decode_serving", "B_per_gpu": B, "Hq": HQ, "Hv": HV, "dk": D, "dv": D,
            "state_bytes_per_gpu": B * HV * D * D * 4, "distinct_steps": N_DISTINCT_STEPS,
            "bytes_per_step_per_gpu": BYTES_PER_STEP, "parallelism": f"batch-sharded x{n_gpus}, no collective",
            "l2": "state (512 MiB) exceeds L2 (126 MB); no flush needed"}


# --------------------------------------------------------------------------- B200 arm
def make_device_steps(torch, dev, seed):
    """64 decode steps' inputs with the workload's distributions, generated on the device."""
    gen = torch.Generator(device=dev).manual_seed(seed)
    n = N_DISTINCT_STEPS
    q = torch.randn(n, B, HQ, D, device=dev, generator=gen)
    q = (q / q.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
    k = torch.randn(n, B, HQ, D, device=dev, generator=gen)
    k = (k / k.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
    v = torch.randn(n, B, HV, D, device=dev, generator=gen).to(torch.bfloat16)
    g = -torch.nn.functional.softplus(torch.randn(n, B, HV, device=dev, generator=gen))
    beta = torch.sigmoid(torch.randn(n, B, HV, device=dev, generator=gen))
    state = torch.randn(B, HV, D, D, device=dev, generator=gen) * 0.02
    return state, q, k, v, g, beta


def run_b200(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the operators have no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from cuda_agent_b200 import capi, load_extension
    ext = load_extension()
    capi.lib()

    state, q, k, v, g, beta = make_device_steps(torch, dev, 1235 + rank)
    out = torch.empty(B, HV, D, device=dev)
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    windows = []

    # ---- device-resident timing through the C ABI
    def step(i):
        j = i % N_DISTINCT_STEPS
        capi.gdn_decode(state, out, q[j], k[j], v[j], g[j], beta[j], args.config)

    for i in range(args.warmup):
        step(i)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.monotonic()
    ev0.record(stream)
    for i in range(args.steps):
        step(i)
    ev1.record(stream)
    barrier()
    windows.append((w0, time.monotonic()))
    ms_total = ev0.elapsed_time(ev1)
    assert bool(torch.isfinite(out).all()), "non-finite decode output"

    # ---- the same loop recorded as CUDA graphs of N_DISTINCT_STEPS launches each (reported beside the headline)
    graph_ms = None
    if args.graph:
        from cuda_agent_b200.graphs import GdnDecodeGraph
        gdn_graph = GdnDecodeGraph(state, out, q, k, v, g, beta, args.config)
        replays = max(1, args.steps // N_DISTINCT_STEPS)
        gdn_graph.replay()
        barrier()
        w0 = time.monotonic()
        ev0.record(stream)
        for _ in range(replays):
            gdn_graph.replay()
        ev1.record(stream)
        barrier()
        windows.append((w0, time.monotonic()))
        graph_ms = ev0.elapsed_time(ev1) / (replays * N_DISTINCT_STEPS)

    # ---- end to end through the extension op, host buffers in, host buffer out
    pin = lambda t: t.cpu().pin_memory()
    hq, hk, hv_, hg, hb = pin(q), pin(k), pin(v), pin(g), pin(beta)
    ho = torch.empty(2, B, HV, D).pin_memory()
    dq = [torch.empty_like(q[0]) for _ in range(2)]
    dk = [torch.empty_like(k[0]) for _ in range(2)]
    dv = [torch.empty_like(v[0]) for _ in range(2)]
    dg = [torch.empty_like(g[0]) for _ in range(2)]
    db = [torch.empty_like(beta[0]) for _ in range(2)]
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]

    def e2e_loop(n):
        """Double-buffered: inputs of step i+1 upload while step i computes; o downloads behind it."""
        def upload(i):
            s, j = i % 2, i % N_DISTINCT_STEPS
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(in_free[s])
                dq[s].copy_(hq[j], non_blocking=True); dk[s].copy_(hk[j], non_blocking=True)
                dv[s].copy_(hv_[j], non_blocking=True); dg[s].copy_(hg[j], non_blocking=True)
                db[s].copy_(hb[j], non_blocking=True)
                in_ready[s].record(copy_in)
        for e in in_free:
            e.record(stream)
        upload(0)
        for i in range(n):
            s = i % 2
            if i + 1 < n:
                upload(i + 1)
            stream.wait_event(in_ready[s])
            o, _ = ext.gdn_decode_forward(state, dq[s], dk[s], dv[s], dg[s], db[s], args.config)
            in_free[s].record(stream)
            done = torch.cuda.Event()
            done.record(stream)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                ho[s].copy_(o, non_blocking=True)
                o.record_stream(copy_out)
                out_done[s].record(copy_out)
        copy_out.synchronize()

    for e in out_done:
        e.record(copy_out)
    e2e_loop(min(args.warmup, 16))
    barrier()
    w0 = time.monotonic()
    t0 = time.perf_counter()
    e2e_loop(args.steps)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    windows.append((w0, time.monotonic()))
    sampler.stop()

    # ---- max over ranks
    times = torch.tensor([ms_total, e2e_s * 1e3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = float(times[0]), float(times[1])
    ms_per_step = ms_total / args.steps
    value = BYTES_PER_STEP * world / (ms_per_step * 1e-3) / 1e9
    e2e_value = BYTES_PER_STEP * world / (e2e_ms / args.steps * 1e-3) / 1e9
    per_gpu = value / world

    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        peak, peak_src = float(json.loads(peaks_file.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = FALLBACK_HBM_GBS, "fallback"

    if rank == 0:
        line = {
            "metric": "gdn_decode_gbps", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(world),
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": H2D_BYTES * world,
                    "d2h_bytes_per_step": D2H_BYTES * world, "ms_per_step": round(e2e_ms / args.steps, 5),
                    "api": "cuda_extension.gdn_decode_forward"},
            "gpu_launches": args.steps,
            "roofline": {"bound": "hbm", "kernel": "gdn_decode_v8_kernel<8>", "achieved": round(per_gpu, 2),
                         "peak": peak, "unit": "GB/s", "frac": round(per_gpu / peak, 4),
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "algorithmic_bytes": BYTES_PER_STEP,
                         "peak_source": peak_src},
            "clocks": sampler.summary(windows),
        }
        if graph_ms is not None:
            line["cuda_graph"] = {"ms_per_step": round(graph_ms, 5), "value": round(BYTES_PER_STEP / graph_ms / 1e6, 2),
                                  "unit": "GB/s per GPU", "launches_per_graph": N_DISTINCT_STEPS}
        if world == 1 and not args.no_cpu_baseline:
            gbs, dt, sample, threads = time_oracle_cpu(n_steps=20, n_warmup=1, budget_s=15.0)
            line["cpu_baseline"] = {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": sample, "ms_per_step_sample": round(dt * 1e3, 3)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_moe(args):
    """Secondary line: the FP8 MoE layer of 4096 tokens (hidden 2048, intermediate 1024, 64 experts, top-6).

    value = grouped-GEMM FLOP (6*T*k*H*I) / time of the two grouped GEMM kernels; e2e = the same FLOP
    over the whole layer through cuda_extension.moe_forward with x coming from pinned host memory and
    the output going back. Weights (403 MB) exceed L2, so no flush is needed between steps."""
    import torch
    from cuda_agent_b200.benchmarks import MoeWorkload, time_cuda
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    wl = MoeWorkload(dev)
    steps, warmup = min(args.steps, 200), max(3, min(args.warmup, 20))
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    w0 = time.monotonic()
    ms_gemm = time_cuda(lambda: wl.gemm_step(args.config), steps, warmup)
    ms_layer = time_cuda(lambda: wl.layer_step(config=args.config), steps, warmup)
    hx = wl.x.cpu().pin_memory()
    ho = torch.empty_like(hx).pin_memory()
    dx = torch.empty_like(wl.x)

    def e2e_step():
        dx.copy_(hx, non_blocking=True)
        ho.copy_(wl.layer_step(dx, args.config), non_blocking=True)
    ms_e2e = time_cuda(e2e_step, steps, warmup)
    windows = [(w0, time.monotonic())]
    sampler.stop()
    assert wl.status.cpu().tolist() == [0, 0]
    tflops = wl.gemm_flops / (ms_gemm * 1e-3) / 1e12
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        peak = 2.0 * float(json.loads(peaks_file.read_text())["bf16_tflops"])
        src = "2 x measured bf16 burst (MEASURED_PEAKS.json bf16_tflops); nominal fp8 dense 4500"
    else:
        peak, src = 2.0 * 1590.0, "2 x fallback bf16 1590; nominal fp8 dense 4500"
    line = {
        "metric": "moe_fp8_grouped_gemm_tflops", "value": round(tflops, 2), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms_gemm, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
        "config": {"workload": "moe_fp8_layer", "T": wl.T, "H": wl.H, "I": wl.I, "E": wl.E, "k": wl.k,
                   "gemm_flops": wl.gemm_flops, "min_bytes": wl.min_bytes,
                   "l2": "expert weights (403 MB) exceed L2 (126 MB); no flush needed"},
        "layer_ms": round(ms_layer, 5),
        "e2e": {"value": round(wl.gemm_flops / (ms_e2e * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": hx.numel() * 2, "d2h_bytes_per_step": ho.numel() * 2,
                "ms_per_step": round(ms_e2e, 5), "api": "cuda_extension.moe_forward"},
        "gpu_launches": 2 * steps,
        "roofline": {"bound": "tensor", "kernel": "moe_gemm_fp8_kernel<0> + <1>", "achieved": round(tflops, 2),
                     "peak": peak, "unit": "TFLOP/s", "frac": round(tflops / peak, 4), "traffic": None,
                     "peak_source": src},
        "clocks": sampler.summary(windows),
    }
    print(json.dumps(line), flush=True)


def run_mla(args):
    """Secondary line: sparse MLA decode, 64 sequences x 128 heads, 2048 selected rows of a 2.4 GB cache.

    value = sequences (one new token each) per second with everything in HBM; e2e = the same through
    cuda_extension.mla_sparse_decode_forward with q / idx / seq_len from pinned host memory and the output
    back (the KV cache is resident, as in serving). The cache (2.4 GB) exceeds L2; the 2048 rows a step
    touches per sequence are 151 MB in total, also above L2, so no flush is needed."""
    import torch
    import torch.distributed as dist
    from cuda_agent_b200.benchmarks import MlaWorkload, time_cuda
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    wl = MlaWorkload(dev, seed=1236 + rank)
    steps, warmup = min(args.steps, 200), max(3, min(args.warmup, 20))
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    w0 = time.monotonic()

    def timed(fn):
        """ms per call: CUDA events between barriers, max over ranks."""
        if world > 1:
            dist.barrier()
        t = torch.tensor([time_cuda(fn, steps, warmup)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    ms = timed(lambda: wl.step(args.nsplit, args.config))
    hq, hidx, hlen = wl.q.cpu().pin_memory(), wl.idx.cpu().pin_memory(), wl.seq_len.cpu().pin_memory()
    ho = torch.empty(wl.out.shape, dtype=torch.bfloat16).pin_memory()
    dq, didx, dlen = torch.empty_like(wl.q), torch.empty_like(wl.idx), torch.empty_like(wl.seq_len)

    def e2e_step():
        dq.copy_(hq, non_blocking=True); didx.copy_(hidx, non_blocking=True); dlen.copy_(hlen, non_blocking=True)
        ho.copy_(wl.api_step(dq, didx, dlen), non_blocking=True)
    ms_e2e = timed(e2e_step)
    windows = [(w0, time.monotonic())]
    sampler.stop()
    assert int(wl.status) == 0
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    peaks = json.loads(peaks_file.read_text()) if peaks_file.exists() else {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": 1590.0}
    t_roof = max(wl.bytes / (peaks["hbm_gbs"] * 1e9), wl.flops / (peaks["bf16_tflops"] * 1e12))
    gbs = wl.bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": "sparse_mla_decode_tok_per_s", "value": round(wl.B * world / (ms * 1e-3), 1), "unit": "tok/s",
        "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 (fp32 softmax and accumulation)", "data": "synthetic",
        "config": {"workload": "sparse_mla_decode", "B_per_gpu": wl.B, "heads": wl.Hh, "S": wl.S, "topk": wl.topk,
                   "nsplit": args.nsplit, "bytes": wl.bytes, "flops": wl.flops,
                   "l2": "rows touched per step (151 MB) and the cache (2.4 GB) exceed L2; no flush needed"},
        "e2e": {"value": round(wl.B * world / (ms_e2e * 1e-3), 1), "unit": "tok/s",
                "h2d_bytes_per_step": (hq.numel() * 2 + hidx.numel() * 4 + hlen.numel() * 4) * world,
                "d2h_bytes_per_step": ho.numel() * 2 * world, "ms_per_step": round(ms_e2e, 5),
                "api": "cuda_extension.mla_sparse_decode_forward"},
        "gpu_launches": steps * (1 if args.nsplit == 1 else 2),
        "roofline": {"bound": "hbm", "kernel": "mla_sparse_decode_pair_kernel", "achieved": round(gbs, 1),
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4), "traffic": None,
                     "roofline_time_us": round(t_roof * 1e6, 2), "frac_of_roofline_time": round(t_roof / (ms * 1e-3), 4),
                     "peak_source": "MEASURED_PEAKS.json (hbm_gbs; bf16_tflops for the compute side)"},
        "clocks": sampler.summary(windows),
    }
    print(json.dumps(line), flush=True)


def run_moe_ep(args):
    """Secondary line: the expert-parallel FP8 MoE layer (8192 tokens per GPU, H 7168, I 2048, 256 experts
    over the ranks, top-8 group-limited sigmoid routing, one shared expert). Launch with torchrun for N > 1.
    value = GEMM FLOP of all ranks / max-over-ranks layer time (CUDA events around the whole layer call,
    all-to-all exchanges included). e2e adds the host round trip of x and the output."""
    import torch
    import torch.distributed as dist
    from cuda_agent_b200.benchmarks import MoeEpWorkload
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    wl = MoeEpWorkload(dev, rank, world, micro_batches=args.micro_batches, gemm_ctas=args.config,
                       dedup=False if args.no_dedup else None)
    steps, warmup = min(args.steps, 30), max(3, min(args.warmup, 5))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    sampler = ClockSampler(local_rank)
    sampler.start()
    w0 = time.monotonic()
    ms = timed(wl.step)
    hx = wl.x.cpu().pin_memory()
    ho = torch.empty_like(hx).pin_memory()
    dx = torch.empty_like(wl.x)

    def e2e_step():
        dx.copy_(hx, non_blocking=True)
        ho.copy_(wl.step(dx), non_blocking=True)
    ms_e2e = timed(e2e_step)
    windows = [(w0, time.monotonic())]
    sampler.stop()
    assert wl.ops.status.cpu().tolist() == [0, 0, 0, 0]
    if rank == 0:
        tflops = wl.flops_per_gpu * world / (ms * 1e-3) / 1e12
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        peak = 2.0 * (float(json.loads(peaks_file.read_text())["bf16_tflops"]) if peaks_file.exists() else 1590.0)
        line = {
            "metric": "moe_ep_fp8_layer_tflops", "value": round(tflops, 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
            "config": {"workload": "moe_ep_layer", "T_per_gpu": wl.T, "H": wl.H, "I": wl.I, "E": wl.E, "k": wl.k,
                       "experts_per_gpu": wl.E // world, "shared_experts": 1, "flops_per_gpu": wl.flops_per_gpu,
                       "parallelism": f"ep{world}, NCCL all-to-all dispatch/return",
                       "l2": "expert weights (>= 1.4 GB per GPU) exceed L2; no flush needed"},
            "e2e": {"value": round(wl.flops_per_gpu * world / (ms_e2e * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                    "h2d_bytes_per_step": hx.numel() * 2 * world, "d2h_bytes_per_step": ho.numel() * 2 * world,
                    "ms_per_step": round(ms_e2e, 4), "api": "cuda_agent_b200.ep.ep_moe_forward"},
            "gpu_launches": steps * 14,
            "roofline": {"bound": "tensor", "kernel": "moe_gemm_fp8_kernel (layer time incl. exchanges)",
                         "achieved": round(tflops / world, 2), "peak": peak, "unit": "TFLOP/s",
                         "frac": round(tflops / world / peak, 4), "traffic": None,
                         "peak_source": "2 x measured bf16 burst; per GPU"},
            "clocks": sampler.summary(windows),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.workload == "moe_ep" and args.impl != "reference":
        return run_moe_ep(args)
    if args.workload == "moe" and args.impl != "reference":
        return run_moe(args)
    if args.workload == "mla" and args.impl != "reference":
        return run_mla(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
