#!/usr/bin/env python3
"""Timing loop: eager ``Model``, ``torch.compile(Model)`` and ``ModelNew``.

Command line and result line follow the reference loop
(agent_workdir/utils/profiling.py:29-39, :76-82):

  python3 -m utils.profiling [--iters N] [--single-run targets]
  -> "Torch Baseline: …us, Torch Compile: …us, CUDA Extension: …us"

and so does the reference metric: the sum of the device time of every CUDA
event ``torch.profiler`` records, divided by the iterations (lines 70-73), after
5 warm-up calls (line 109) on one fixed set of inputs (lines 51-55).
``--single-run`` runs the named targets once with no profiler attached, which is
where an external profiler hooks in (lines 85-96).

Added: ``--events`` also times each target with CUDA events around the whole
loop (wall time on the stream, launch gaps included); ``--no-compile`` skips the
``torch.compile`` column (printed as nan) for boxes without a working inductor;
``--json PATH`` writes the numbers to a file.
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from ._workspace import add_workspace_args, as_list, load_task, map_tensors

WARMUP_ITERS = 5


def parse_args(argv=None):
    parser = argparse.ArgumentParser(description="Profile cuda_extension vs torch baseline and torch.compile.")
    parser.add_argument("--iters", type=int, default=10, help="Benchmark iterations")
    parser.add_argument("--single-run", type=str,
                        help="Run once for targets: torch_baseline,torch_compile,cuda_extension")
    parser.add_argument("--events", action="store_true", help="also report CUDA-event wall time")
    parser.add_argument("--no-compile", action="store_true", help="skip the torch.compile column")
    parser.add_argument("--json", type=str, default=None, help="write results to this file")
    add_workspace_args(parser)
    return parser.parse_args(argv)


def initialize_models(model, model_new):
    if not torch.cuda.is_available():
        raise RuntimeError("profiling needs a CUDA device: ModelNew has no CPU path")
    init = as_list(model.get_init_inputs())
    torch_model = model.Model(*init).eval().cuda()
    cuda_model = model_new.ModelNew(*init).eval().cuda()
    cuda_model.load_state_dict(torch_model.state_dict())
    torch_inputs = map_tensors(as_list(model.get_inputs()), lambda t: t.cuda())
    cuda_inputs = map_tensors(torch_inputs, lambda t: t.clone())
    return torch_model, cuda_model, torch_inputs, cuda_inputs


def profiler_time_us(module, inputs, warmup_iters: int, run_iters: int) -> float:
    """Sum of CUDA-event device time per iteration, in microseconds."""
    with torch.no_grad():
        for _ in range(warmup_iters):
            module(*inputs)
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA],
                                    record_shapes=False, with_stack=False) as prof:
            torch.cuda.synchronize()
            for _ in range(run_iters):
                module(*inputs)
            torch.cuda.synchronize()
    total = sum(ev.device_time for ev in prof.events() if ev.device_type.name == "CUDA")
    return total / run_iters


def event_time_us(module, inputs, warmup_iters: int, run_iters: int) -> float:
    """Stream wall time per iteration between two CUDA events, in microseconds."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.no_grad():
        for _ in range(warmup_iters):
            module(*inputs)
        torch.cuda.synchronize()
        start.record()
        for _ in range(run_iters):
            module(*inputs)
        stop.record()
        torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / run_iters


def run_single(targets, torch_model, cuda_model, torch_inputs, cuda_inputs) -> None:
    with torch.no_grad():
        if "torch_baseline" in targets:
            torch_model(*torch_inputs)
        if "torch_compile" in targets:
            torch.compile(torch_model)(*torch_inputs)
        if "cuda_extension" in targets:
            cuda_model(*cuda_inputs)
    torch.cuda.synchronize()
    print("[DONE] single-run completed")


def main(argv=None) -> int:
    args = parse_args(argv)
    model, model_new = load_task(args)
    torch_model, cuda_model, torch_inputs, cuda_inputs = initialize_models(model, model_new)

    if args.single_run:
        targets = [t.strip() for t in args.single_run.split(",") if t.strip()]
        run_single(targets, torch_model, cuda_model, torch_inputs, cuda_inputs)
        return 0

    results = {}
    order = [("cuda_extension", cuda_model, cuda_inputs), ("torch_baseline", torch_model, torch_inputs)]
    if not args.no_compile:
        order.append(("torch_compile", torch.compile(torch_model), torch_inputs))
    for name, module, inputs in order:
        results[name] = profiler_time_us(module, inputs, WARMUP_ITERS, args.iters)
        if args.events:
            results[name + "_event_us"] = event_time_us(module, inputs, WARMUP_ITERS, args.iters)
    compile_us = results.get("torch_compile", math.nan)
    print(f"Torch Baseline: {results['torch_baseline']:.3f}us, "
          f"Torch Compile: {compile_us:.3f}us, "
          f"CUDA Extension: {results['cuda_extension']:.3f}us")
    if args.events:
        print("CUDA-event wall time per iteration: " + ", ".join(
            f"{k[:-9]}={v:.3f}us" for k, v in results.items() if k.endswith("_event_us")))
    if args.json:
        with open(args.json, "w") as fh:
            json.dump({"iters": args.iters, "warmup": WARMUP_ITERS, **results}, fh)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
