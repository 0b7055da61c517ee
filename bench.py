#!/usr/bin/env python3
"""Benchmark of the three decode/inference hot paths; the headline is Gated DeltaNet decode in GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload all|gdn|moe|mla|moe_ep]

One JSON line on rank 0. Headline workload ("gdn_decode_serving"): B=256 sequences per GPU, 16 q/k heads
shared by groups of 2 across 32 value heads, dk=dv=128, fp32 state of 512 MiB per GPU. One step is one decode
step (one kernel launch over the whole batch) with that step's own q/k/v/g/beta, taken in turn from 64
pre-generated seeded steps. Algorithmic bytes per step per GPU: state read + write 2*536870912, q and k
2*1048576, v 2097152, g and beta 2*32768, o 4194304 = 1082195968. Consecutive steps walk the state in alternating
directions (--gdn-walk zigzag, the default: the op's config bit 4 on odd steps), so a step starts on the rows the
previous one wrote last and finds about 80 MB of them in L2; --gdn-walk forward walks every step the same way.

Keys of the line:
  value        GB/s over all GPUs with every input already in HBM (CUDA events, max over ranks)
  e2e          same metric through cuda_extension.gdn_decode_forward with the step's inputs coming from
               pinned host memory and o going back to it, copies inside the timed region (the 512 MiB
               state lives on the GPU between steps, as it does in a serving process)
  roofline     the decode kernel against measured HBM copy bandwidth
  cpu_baseline the eager oracle on this box's host cores (a reported baseline; N=1 only)
  clocks       SM clock and throttle reasons sampled during the timed regions
  secondary    with --workload all (the default), one record per other path, each with its own value,
               ms_per_step, e2e, roofline and (N=1) cpu_baseline:
                 moe     FP8 MoE layer, 4096 tokens, 64 experts, top-6 (one GPU by definition: N=1 only)
                 mla     top-2048 sparse MLA decode, 64 sequences x 128 heads per GPU (batch-sharded)
                 moe_ep  expert-parallel FP8 MoE layer, 8192 tokens per GPU, 256 experts over the ranks,
                         with `parity` = rel-L2 of 256 tokens of every rank against the eager oracle's functions

Every timed region lasts at least MIN_REGION_S seconds: when the requested --steps finish sooner, the
region is repeated with more steps, and the number of steps actually timed is what the line reports
("steps"; the request is kept in "steps_requested").

With N > 1 GDN and MLA are sharded by batch with no collective (every rank runs the same per-GPU workload:
weak scaling); the expert-parallel layer exchanges rows between the ranks. NCCL carries the barrier and
the max over ranks.

``--impl reference`` times the eager CPU oracles (the reference's torch-eager path for these operators)
on all host cores instead; rank 0 only. The rates it prints are those of one host and do not depend on N.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MIN_REGION_S = 0.5
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
NOMINAL_FP8_TFLOPS = 4500.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu captures of each kernel at
# these workloads (the summaries under profiles/ give the commands).
NCU_TRAFFIC = {
    "gdn_decode_v8_kernel<8>": 946561229,            # zig-zag loop, caches not flushed between launches
    "gdn_decode_v8_kernel<8> forward": 1081152256,  # every step walked forwards
    "moe_gemm_fp8_kernel<0> + <1>": 355400000 + 246100000,
    "mla_sparse_decode_pair_kernel": 166300000,
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=640)
    ap.add_argument("--warmup", type=int, default=64)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--config", type=int, default=0, help="launcher variant passed to the op")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graph", action="store_true",
                    help="gdn: also time the loop recorded as CUDA graphs (extra key \"cuda_graph\")")
    ap.add_argument("--workload", choices=["all", "gdn", "moe", "mla", "moe_ep"], default="all",
                    help="all = headline GDN line with the other paths under \"secondary\"; a single name = "
                         "that path alone as the line")
    ap.add_argument("--ep-mode", choices=["peer", "nccl"], default="peer",
                    help="moe_ep: rows pushed into the peers' receive buffers by the kernels themselves (peer) "
                         "or exchanged with NCCL all-to-all calls (nccl)")
    ap.add_argument("--nsplit", type=int, default=0, help="mla: splits of the selected rows (0 = the op's choice)")
    ap.add_argument("--min-region-s", type=float, default=MIN_REGION_S)
    ap.add_argument("--gdn-walk", choices=["zigzag", "forward"], default="zigzag",
                    help="gdn: alternate the direction in which a step walks the state (each step starts on the rows "
                         "the previous one left in L2) or always walk it forwards")
    ap.add_argument("--ep-tokens", type=int, default=8192,
                    help="moe_ep: tokens per GPU (the benchmark's figure is 8192; smaller values are for profiler captures)")
    ap.add_argument("--ep-gemm-ctas", type=int, default=0,
                    help="moe_ep: persistent CTAs of the grouped GEMMs (0 = the launcher's choice)")
    ap.add_argument("--ep-experts", type=int, default=256,
                    help="moe_ep: routed experts over all ranks, a multiple of 8 groups (benchmark: 256)")
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


def load_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        p = json.loads(f.read_text())
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "source": "fallback"}


# --------------------------------------------------------------------------- run context
class Ctx:
    """Ranks, barrier, and timed regions of at least `min_s` seconds whose length every rank agrees on."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device (the operators have no CPU path)")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.sampler = ClockSampler(self.local_rank)
        self.sampler.start()
        self.windows = []
        self.peaks = load_peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        t = self.torch.tensor([value], device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t)

    def timed(self, step, steps, warmup, wall=False, run_n=None):
        """(ms per step as the max over ranks, steps timed). `step(i)` enqueues step i; with run_n given, the
        region is run_n(n) (a pipelined loop that ends synchronised) and is timed by the host clock, otherwise
        by CUDA events on the current stream. The region is repeated with more steps until it lasts min_s."""
        torch = self.torch
        stream = torch.cuda.current_stream()

        def region(n):
            self.barrier()
            w0 = time.monotonic()
            if run_n is not None:
                t0 = time.perf_counter()
                run_n(n)
                torch.cuda.synchronize()
                ms = (time.perf_counter() - t0) * 1e3
            else:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for i in range(n):
                    step(i)
                e1.record(stream)
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1)
            self.barrier()
            self.windows.append((w0, time.monotonic()))
            return self.max_over_ranks(ms)

        if run_n is not None:
            run_n(max(3, warmup))
        else:
            for i in range(max(3, warmup)):
                step(i)
        n = max(1, steps)
        ms = region(n)
        min_ms = self.args.min_region_s * 1e3
        if ms < min_ms:
            n = int(math.ceil(n * min_ms * 1.1 / max(ms, 1e-3)))
            ms = region(n)
        return ms / n, n

    def finish(self):
        self.sampler.stop()
        clocks = self.sampler.summary(self.windows)
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()
        return clocks


# --------------------------------------------------------------------------- the four paths (B200 arm)
def gdn_record(ctx: Ctx, cpu_baseline: bool):
    import bench_workloads as bw
    args, torch = ctx.args, ctx.torch
    wl = bw.GdnWorkload(ctx.dev, 1235 + ctx.rank)
    zz = args.gdn_walk == "zigzag"
    ms, n = ctx.timed(lambda i: wl.step(i, args.config, zz), args.steps, args.warmup)
    assert bool(torch.isfinite(wl.out).all()), "non-finite decode output"
    # the other walk, for the record: with every step walked forwards nothing of the state is found in L2
    other_ms, _ = ctx.timed(lambda i: wl.step(i, args.config, not zz), args.steps, 3)
    graph = None
    if args.graph:
        from cuda_agent_b200.graphs import GdnDecodeGraph
        g = GdnDecodeGraph(wl.state, wl.out, wl.q, wl.k, wl.v, wl.g, wl.beta, args.config, zz)
        gms, gn = ctx.timed(lambda i: g.replay(), max(1, args.steps // wl.N_DISTINCT), 1)
        graph = {"ms_per_step": round(gms / wl.N_DISTINCT, 5), "unit": "GB/s per GPU",
                 "value": round(wl.bytes_per_step / (gms / wl.N_DISTINCT) / 1e6, 2), "launches_per_graph": wl.N_DISTINCT}
    pipe = wl.make_e2e(args.config, zz)
    e2e_ms, e2e_n = ctx.timed(None, args.steps, min(args.warmup, 16), run_n=pipe.run)
    world = ctx.world
    per_gpu = wl.bytes_per_step / (ms * 1e-3) / 1e9
    peak = ctx.peaks["hbm_gbs"]
    kernel = "gdn_decode_v8_kernel<8>"
    rec = {
        "metric": "gdn_decode_gbps", "value": round(per_gpu * world, 2), "unit": "GB/s", "n_gpus": world,
        "steps": n, "steps_requested": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gdn_decode_serving", "B_per_gpu": wl.B, "Hq": wl.HQ, "Hv": wl.HV, "dk": wl.D,
                   "dv": wl.D, "state_bytes_per_gpu": wl.B * wl.HV * wl.D * wl.D * 4,
                   "distinct_steps": wl.N_DISTINCT, "bytes_per_step_per_gpu": wl.bytes_per_step,
                   "parallelism": f"batch-sharded x{world}, no collective",
                   "l2": "state (512 MiB) exceeds L2 (126 MB); no flush needed" + ("; zig-zag walk: a step starts on the rows the previous step wrote last (about 80 MB still in L2)" if zz else ""),
                   "min_timed_region_s": args.min_region_s},
        "e2e": {"value": round(wl.bytes_per_step * world / (e2e_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
                "h2d_bytes_per_step": wl.h2d_bytes * world, "d2h_bytes_per_step": wl.d2h_bytes * world,
                "ms_per_step": round(e2e_ms, 5), "steps": e2e_n, "api": "cuda_extension.gdn_decode_forward",
                "copies_per_step": "1 host->device (packed q,k,v,g,beta), 1 device->host"},
        "walk": {"timed": args.gdn_walk, "other": "forward" if zz else "zigzag",
                 "other_value": round(wl.bytes_per_step * world / (other_ms * 1e-3) / 1e9, 2),
                 "other_ms_per_step": round(other_ms, 5),
                 "note": "zigzag: consecutive steps walk the state in alternating directions and find about 80 MB "
                         "of it in L2; forward: every step walks it the same way (what a model with many such "
                         "layers would see)"},
        "gpu_launches": n,
        "roofline": {"bound": "hbm", "kernel": kernel, "achieved": round(per_gpu, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(per_gpu / peak, 4), "traffic": NCU_TRAFFIC[kernel if zz else kernel + " forward"],
                     "algorithmic_bytes": wl.bytes_per_step, "peak_source": ctx.peaks["source"] + " hbm_gbs"},
    }
    if graph:
        rec["cuda_graph"] = graph
    if cpu_baseline:
        gbs, dt, sample, threads = bw.cpu_gdn(budget_s=12.0)
        rec["cpu_baseline"] = {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
                               "sample": sample, "ms_per_step_sample": round(dt * 1e3, 3)}
    del wl, pipe
    torch.cuda.empty_cache()
    return rec


def moe_record(ctx: Ctx, cpu_baseline: bool):
    """FP8 MoE layer of 4096 tokens (H 2048, I 1024, 64 experts, top-6) on one GPU. value = grouped-GEMM FLOP
    (6*T*k*H*I) / time of the two grouped GEMM kernels; e2e = the same FLOP over the whole layer through
    cuda_extension.moe_forward with x from pinned host memory and the output back (pipelined)."""
    import bench_workloads as bw
    args, torch = ctx.args, ctx.torch
    wl = bw.MoeWorkload(ctx.dev)
    steps, warmup = min(args.steps, 200), min(args.warmup, 20)
    ms_gemm, n = ctx.timed(lambda i: wl.gemm_step(args.config), steps, warmup)
    ms_layer, _ = ctx.timed(lambda i: wl.layer_step(config=args.config), steps, warmup)
    pipe = wl.make_e2e(args.config)
    ms_e2e, n_e2e = ctx.timed(None, steps, 5, run_n=pipe.run)
    assert wl.status.cpu().tolist() == [0, 0]
    tflops = wl.gemm_flops / (ms_gemm * 1e-3) / 1e12
    peak2 = 2.0 * ctx.peaks["bf16_tflops"]
    try:
        lib_burst, lib_sustained = bw.library_fp8_gemm_tflops(ctx.dev)
    except Exception as exc:                      # a yardstick only: the line stands without it
        lib_burst = lib_sustained = None
        print(f"bench.py: library fp8 yardstick unavailable: {exc}", file=sys.stderr)
    kernel = "moe_gemm_fp8_kernel<0> + <1>"
    rec = {
        "metric": "moe_fp8_grouped_gemm_tflops", "value": round(tflops, 2), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": n, "ms_per_step": round(ms_gemm, 5), "higher_is_better": True,
        "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
        "config": {"workload": "moe_fp8_layer", "T": wl.T, "H": wl.H, "I": wl.I, "E": wl.E, "k": wl.k,
                   "gemm_flops": wl.gemm_flops, "min_bytes": wl.min_bytes,
                   "l2": "expert weights (403 MB) exceed L2 (126 MB); no flush needed"},
        "layer_ms": round(ms_layer, 5),
        "layer_tflops": round(wl.gemm_flops / (ms_layer * 1e-3) / 1e12, 2),
        "e2e": {"value": round(wl.gemm_flops / (ms_e2e * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": wl.h2d_bytes, "d2h_bytes_per_step": wl.d2h_bytes,
                "ms_per_step": round(ms_e2e, 5), "steps": n_e2e, "api": "cuda_extension.moe_forward"},
        "gpu_launches": 2 * n,
        "roofline": {"bound": "tensor", "kernel": kernel, "achieved": round(tflops, 2), "peak": NOMINAL_FP8_TFLOPS,
                     "unit": "TFLOP/s", "frac": round(tflops / NOMINAL_FP8_TFLOPS, 4),
                     "peak_source": "nominal fp8 dense (no measured fp8 figure exists)",
                     "frac_of_2x_measured_bf16": round(tflops / peak2, 4), "peak_2x_measured_bf16": peak2,
                     "library_dense_fp8_8192_cubed_tflops": None if lib_burst is None else
                     {"burst": round(lib_burst, 1), "sustained": round(lib_sustained, 1),
                      "frac_of_sustained": round(tflops / lib_sustained, 4)},
                     "traffic": NCU_TRAFFIC[kernel]},
    }
    if cpu_baseline:
        tf, dt, sample, threads = bw.cpu_moe()
        rec["cpu_baseline"] = {"value": round(tf, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port",
                               "sample": sample, "s_per_layer": round(dt, 3)}
    del wl, pipe
    torch.cuda.empty_cache()
    return rec


def mla_record(ctx: Ctx, cpu_baseline: bool):
    """Sparse MLA decode, 64 sequences x 128 heads per GPU, 2048 selected rows of a 2.4 GB cache. value =
    sequences (one new token each) per second with everything in HBM; e2e = the same through
    cuda_extension.mla_sparse_decode_forward with q / idx / seq_len from pinned host memory and the output
    back (the KV cache is resident, as in serving)."""
    import bench_workloads as bw
    args, torch = ctx.args, ctx.torch
    wl = bw.MlaWorkload(ctx.dev, seed=1236 + ctx.rank)
    steps, warmup = min(args.steps, 200), min(args.warmup, 20)
    nsplit = args.nsplit if args.nsplit > 0 else 1
    ms, n = ctx.timed(lambda i: wl.step(nsplit, args.config), steps, warmup)
    pipe = wl.make_e2e(args.nsplit, args.config)
    ms_e2e, n_e2e = ctx.timed(None, steps, 5, run_n=pipe.run)
    assert int(wl.status) == 0
    world = ctx.world
    peaks = ctx.peaks
    t_roof = max(wl.bytes / (peaks["hbm_gbs"] * 1e9), wl.flops / (peaks["bf16_tflops"] * 1e12))
    gbs = wl.bytes / (ms * 1e-3) / 1e9
    kernel = "mla_sparse_decode_pair_kernel"
    rec = {
        "metric": "sparse_mla_decode_tok_per_s", "value": round(wl.B * world / (ms * 1e-3), 1), "unit": "tok/s",
        "n_gpus": world, "steps": n, "ms_per_step": round(ms, 5), "higher_is_better": True, "scaling": "weak",
        "dtype": "bf16 (fp32 softmax and accumulation)", "data": "synthetic",
        "config": {"workload": "sparse_mla_decode", "B_per_gpu": wl.B, "heads": wl.Hh, "S": wl.S, "topk": wl.topk,
                   "nsplit": nsplit, "bytes": wl.bytes, "flops": wl.flops,
                   "parallelism": f"batch-sharded x{world}, no collective",
                   "l2": "rows touched per step (151 MB) and the cache (2.4 GB) exceed L2; no flush needed"},
        "e2e": {"value": round(wl.B * world / (ms_e2e * 1e-3), 1), "unit": "tok/s",
                "h2d_bytes_per_step": wl.h2d_bytes * world, "d2h_bytes_per_step": wl.d2h_bytes * world,
                "ms_per_step": round(ms_e2e, 5), "steps": n_e2e, "api": "cuda_extension.mla_sparse_decode_forward"},
        "gpu_launches": n * (1 if nsplit == 1 else 2),
        "roofline": {"bound": "hbm", "kernel": kernel, "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4), "traffic": NCU_TRAFFIC[kernel],
                     "roofline_time_us": round(t_roof * 1e6, 2), "frac_of_roofline_time": round(t_roof / (ms * 1e-3), 4),
                     "peak_source": peaks["source"] + " hbm_gbs; bf16_tflops for the compute side"},
    }
    if cpu_baseline:
        tps, dt, sample, threads = bw.cpu_mla(wl)
        rec["cpu_baseline"] = {"value": round(tps, 2), "unit": "tok/s", "cores": threads, "kind": "port",
                               "sample": sample, "s_per_sequence": round(dt, 4)}
    del wl, pipe
    torch.cuda.empty_cache()
    return rec


def moe_ep_record(ctx: Ctx, cpu_baseline: bool):
    """Expert-parallel FP8 MoE layer (8192 tokens per GPU, H 7168, I 2048, 256 experts over the ranks, top-8
    group-limited sigmoid routing, one shared expert). value = GEMM FLOP of all ranks / max-over-ranks layer
    time (CUDA events around the whole layer call, exchanges included). e2e adds the host round trip of x and
    the output (pipelined)."""
    import bench_workloads as bw
    args, torch = ctx.args, ctx.torch
    wl = bw.MoeEpWorkload(ctx.dev, ctx.rank, ctx.world, T=args.ep_tokens, E=args.ep_experts, mode=args.ep_mode,
                          gemm_ctas=args.ep_gemm_ctas)
    steps, warmup = min(args.steps, 30), min(args.warmup, 5)
    ctx.barrier()                     # every rank's weights and exchange buffers exist before the first call
    out = wl.step()
    torch.cuda.synchronize()
    # checker leg, untimed: every rank compares its own first tokens with the oracle; rank 0 reports the worst
    mine = wl.parity(out, min(256, wl.T))
    parity = mine
    if ctx.world > 1:
        every = [None] * ctx.world
        ctx.dist.all_gather_object(every, mine)
        parity = {"rel_l2": max(p["rel_l2"] for p in every), "tokens": sum(p["tokens"] for p in every),
                  "tokens_routed_differently": sum(p["tokens_routed_differently"] for p in every),
                  "rel_l2_identically_routed": max(p["rel_l2_identically_routed"] for p in every),
                  "rel_l2_per_rank": [p["rel_l2"] for p in every]}
    del out
    ctx.barrier()
    ms, n = ctx.timed(lambda i: wl.step(), steps, warmup)
    pipe = wl.make_e2e()
    ms_e2e, n_e2e = ctx.timed(None, steps, 3, run_n=pipe.run)
    status = wl.layer.status_codes()
    assert not any(status), f"a kernel of the layer gave up a bounded wait or flagged its input: {status}"
    world = ctx.world
    tflops = wl.flops_per_gpu * world / (ms * 1e-3) / 1e12
    peak2 = 2.0 * ctx.peaks["bf16_tflops"]
    rec = {
        "metric": "moe_ep_fp8_layer_tflops", "value": round(tflops, 2), "unit": "TFLOP/s", "n_gpus": world,
        "steps": n, "ms_per_step": round(ms, 4), "layer_ms_max_over_ranks": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
        "config": {"workload": "moe_ep_layer", "T_per_gpu": wl.T, "H": wl.H, "I": wl.I, "E": wl.E, "k": wl.k,
                   "experts_per_gpu": wl.E // world, "shared_experts": 1, "flops_per_gpu": wl.flops_per_gpu,
                   "parallelism": f"ep{world}, " + wl.layer.describe(),
                   "l2": "expert weights (>= 1.4 GB per GPU) exceed L2; no flush needed"},
        "parity": dict(parity or {}, tolerance=2e-2,
                       against="oracle/moe/model.py functions on every rank's first 256 tokens (worst rank "
                               "reported), on the GPU, untimed"),
        "e2e": {"value": round(wl.flops_per_gpu * world / (ms_e2e * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": wl.h2d_bytes * world, "d2h_bytes_per_step": wl.d2h_bytes * world,
                "ms_per_step": round(ms_e2e, 4), "steps": n_e2e, "api": "cuda_agent_b200.ep layer.forward"},
        "gpu_launches": n * wl.layer.launches_per_call(),
        "roofline": {"bound": "tensor", "kernel": "moe_gemm_fp8_kernel (layer time incl. exchanges)",
                     "achieved": round(tflops / world, 2), "peak": NOMINAL_FP8_TFLOPS, "unit": "TFLOP/s",
                     "frac": round(tflops / world / NOMINAL_FP8_TFLOPS, 4),
                     "peak_source": "nominal fp8 dense, per GPU",
                     "frac_of_2x_measured_bf16": round(tflops / world / peak2, 4), "traffic": None},
    }
    assert parity["rel_l2_identically_routed"] <= 2e-2, f"expert-parallel layer off the oracle: {parity}"
    if cpu_baseline:
        tf, dt, sample, threads = bw.cpu_moe_ep()
        rec["cpu_baseline"] = {"value": round(tf, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port",
                               "sample": sample, "s_sample": round(dt, 3),
                               "s_per_layer_extrapolated": round(wl.flops_per_gpu / (tf * 1e12), 2)}
    wl.layer.close()
    del wl, pipe
    torch.cuda.empty_cache()
    return rec


RECORDS = {"gdn": gdn_record, "moe": moe_record, "mla": mla_record, "moe_ep": moe_ep_record}


def run_b200(args):
    from cuda_agent_b200 import capi, load_extension
    load_extension()
    capi.lib()
    ctx = Ctx(args)
    cpu = ctx.world == 1 and not args.no_cpu_baseline
    head = "gdn" if args.workload == "all" else args.workload
    if head == "moe" and ctx.world > 1:
        raise SystemExit("bench.py: --workload moe is the one-GPU layer; the expert-parallel one is moe_ep")
    line = RECORDS[head](ctx, cpu)
    line.setdefault("n_gpus", ctx.world)
    line.setdefault("scaling", "weak")
    line.setdefault("vs_baseline", None)
    line.setdefault("warmup", max(3, args.warmup))
    if args.workload == "all":
        sec = {}
        names = (["moe"] if ctx.world == 1 else []) + ["mla", "moe_ep"]
        for name in names:
            # a path that fails (on every rank alike) is reported under its name; the other paths keep their records
            try:
                sec[name] = RECORDS[name](ctx, cpu)
            except Exception as exc:  # noqa: BLE001
                sec[name] = {"error": f"{type(exc).__name__}: {exc}"[:400], "gpu_launches": 0}
                ctx.torch.cuda.synchronize()
        line["secondary"] = sec
        line["gpu_launches"] += sum(r["gpu_launches"] for r in sec.values())
    line["clocks"] = ctx.finish()
    if ctx.rank == 0:
        print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- reference arm
def run_reference(args):
    """The eager oracles on all host cores (the reference's torch-eager CPU path for these operators; kind
    "port" because the reference ships no implementation of them). Rank 0 only. The figures are rates of one
    host: they stand for one box's CPU whatever --gpus says."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import bench_workloads as bw
    which = args.workload
    secondary = {}

    def gdn():
        gbs, dt, sample, threads = bw.cpu_gdn(budget_s=60.0 if which == "all" else 150.0,
                                              n_steps=min(args.steps, 20), n_warmup=max(1, min(args.warmup, 2)))
        return {"metric": "gdn_decode_gbps", "value": round(gbs, 3), "unit": "GB/s", "ms_per_step": round(dt * 1e3, 4),
                "dtype": "f32", "config": {"workload": "gdn_decode_serving", "B_per_gpu": 256, "Hq": 16, "Hv": 32,
                                            "dk": 128, "dv": 128},
                "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample}}

    def moe():
        tf, dt, sample, threads = bw.cpu_moe()
        return {"metric": "moe_fp8_grouped_gemm_tflops", "value": round(tf, 4), "unit": "TFLOP/s",
                "ms_per_step": round(dt * 1e3, 2), "dtype": "f32 on dequantised e4m3",
                "config": {"workload": "moe_fp8_layer", "T": 4096, "H": 2048, "I": 1024, "E": 64, "k": 6},
                "cpu_baseline": {"value": round(tf, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample}}

    def mla():
        import torch

        class HostInputs:          # the oracle's own generator at the workload's shapes, 16 sequences
            pass
        m = bw.load_oracle("mla", {"CAB_MLA_CONFIG": 2})
        gen = torch.Generator().manual_seed(1236)
        n_seq = 16
        q, kv, seq_len, idx = m.make_inputs(n_seq, 128, 32768, 2048, 8192, gen)
        wl = HostInputs()
        wl.q, wl.kv, wl.seq_len, wl.idx, wl.Hh, wl.S, wl.topk = q, kv, seq_len, idx, 128, 32768, 2048
        tps, dt, sample, threads = bw.cpu_mla(wl, n_seq)
        return {"metric": "sparse_mla_decode_tok_per_s", "value": round(tps, 2), "unit": "tok/s",
                "ms_per_step": round(dt * 64 * 1e3, 2), "dtype": "f32 from bf16",
                "config": {"workload": "sparse_mla_decode", "B_per_gpu": 64, "heads": 128, "S": 32768, "topk": 2048},
                "cpu_baseline": {"value": round(tps, 2), "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample}}

    def moe_ep():
        tf, dt, sample, threads = bw.cpu_moe_ep()
        flops = 6 * 8192 * 8 * 7168 * 2048 + 6 * 8192 * 7168 * 2048
        return {"metric": "moe_ep_fp8_layer_tflops", "value": round(tf, 4), "unit": "TFLOP/s",
                "ms_per_step": round(flops / (tf * 1e12) * 1e3, 1), "dtype": "f32 on dequantised e4m3",
                "config": {"workload": "moe_ep_layer", "T_per_gpu": 8192, "H": 7168, "I": 2048, "E": 256, "k": 8},
                "cpu_baseline": {"value": round(tf, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample}}

    fns = {"gdn": gdn, "moe": moe, "mla": mla, "moe_ep": moe_ep}
    line = fns["gdn" if which == "all" else which]()
    if which == "all":
        for name in ("moe", "mla", "moe_ep"):
            secondary[name] = fns[name]()
            secondary[name]["e2e"] = {"value": secondary[name]["value"], "unit": secondary[name]["unit"],
                                      "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    line.update({
        "impl": "reference", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
        "e2e": {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "stands_for": "the rate of this one host's CPU cores; it does not grow with n_gpus",
    })
    if secondary:
        line["secondary"] = secondary
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
