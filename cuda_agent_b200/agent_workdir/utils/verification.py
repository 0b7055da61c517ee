#!/usr/bin/env python3
"""Correctness gate: eager ``Model`` against ``ModelNew`` on the GPU.

Same loop and output lines as the reference gate
(agent_workdir/utils/verification.py:85-99): build both modules on the GPU, copy
the eager module's ``state_dict`` into ``ModelNew`` (strict), run N trials on
fresh inputs from ``get_inputs()``, with every public ``torch.nn.functional``
callable raising while ``ModelNew.forward`` runs, and print ``[PASS] check i/N``
then ``[PASS] verify success``.

What is added, because one ``atol = rtol = 1e-2`` (reference line 35) cannot
express "indices must be identical" or "rel 1e-3 on an fp32 state":
``model.py`` may define ``OUTPUT_POLICY``, a nest shaped like the model's output
whose leaves are

  "exact"          torch.equal (integer outputs: indices, permutations, gathers)
  ("rel", t)       ||a-b||_2 / ||b||_2 <= t  and  |a-b| <= t*max|b| + t*|b|
  ("rel_l2", t)    ||a-b||_2 / ||b||_2 <= t only
  ("atol", t)      |a-b| <= t
  ("close", a, r)  torch.testing.assert_close(atol=a, rtol=r)

Without ``OUTPUT_POLICY`` the reference tolerance applies to every tensor.
"""
from __future__ import annotations

import argparse
from contextlib import contextmanager

import torch
import torch.nn.functional as F

from ._workspace import add_workspace_args, as_list, load_task, map_tensors

DEFAULT_POLICY = ("close", 1e-2, 1e-2)


def compare_tensor(actual: torch.Tensor, expected: torch.Tensor, policy, where: str = "output") -> dict:
    """Raise AssertionError unless `actual` matches `expected` under `policy`; return metrics."""
    assert actual.shape == expected.shape, f"{where}: shape {tuple(actual.shape)} != {tuple(expected.shape)}"
    assert actual.dtype == expected.dtype, f"{where}: dtype {actual.dtype} != {expected.dtype}"
    assert actual.device == expected.device, f"{where}: device {actual.device} != {expected.device}"
    kind = policy if isinstance(policy, str) else policy[0]
    if kind == "exact":
        if not torch.equal(actual, expected):
            bad = (actual != expected)
            raise AssertionError(f"{where}: {int(bad.sum())} of {bad.numel()} elements differ (exact policy)")
        return {"policy": "exact", "mismatches": 0}
    a, e = actual.double(), expected.double()
    assert torch.isfinite(a).all(), f"{where}: non-finite values in the extension output"
    diff = (a - e).abs()
    denom = float(e.norm())
    rel_l2 = float((a - e).norm()) / denom if denom > 0 else float(diff.max())
    metrics = {"policy": kind, "rel_l2": rel_l2, "max_abs": float(diff.max()) if diff.numel() else 0.0}
    if kind in ("rel", "rel_l2"):
        tol = float(policy[1])
        assert rel_l2 <= tol, f"{where}: rel-L2 {rel_l2:.3e} > {tol:.1e}"
        if kind == "rel" and diff.numel():
            bound = tol * float(e.abs().max()) + tol * e.abs()
            worst = float((diff - bound).max())
            assert worst <= 0, f"{where}: element error exceeds {tol:.1e}*(max|ref|+|ref|) by {worst:.3e}"
    elif kind == "atol":
        tol = float(policy[1])
        assert metrics["max_abs"] <= tol, f"{where}: max |diff| {metrics['max_abs']:.3e} > {tol:.1e}"
    elif kind == "close":
        torch.testing.assert_close(actual, expected, atol=float(policy[1]), rtol=float(policy[2]))
    else:
        raise ValueError(f"unknown comparison policy {policy!r}")
    return metrics


def check_equal(actual, expected, policy=None, where: str = "output") -> list:
    """Recursive comparison with the container rules of the reference gate (lines 22-37)."""
    assert type(actual) == type(expected), f"{where}: {type(actual)=} != {type(expected)=}"
    if isinstance(actual, (list, tuple)):
        assert len(actual) == len(expected), f"{where}: {len(actual)=} != {len(expected)=}"
        out = []
        for i, (x, y) in enumerate(zip(actual, expected)):
            sub = policy[i] if isinstance(policy, (list, tuple)) and not _is_leaf(policy) else policy
            out += check_equal(x, y, sub, f"{where}[{i}]")
        return out
    if isinstance(actual, dict):
        out = []
        for key, val in expected.items():
            assert key in actual, f"{where}: missing key {key!r}"
            sub = policy.get(key) if isinstance(policy, dict) else policy
            out += check_equal(actual[key], val, sub, f"{where}[{key!r}]")
        return out
    if isinstance(actual, (str, float, int)):
        assert actual == expected, f"{where}: {actual=} != {expected=}"
        return []
    if isinstance(actual, torch.Tensor):
        return [compare_tensor(actual, expected, policy or DEFAULT_POLICY, where)]
    raise TypeError(f"{where}: unsupported output type {type(actual)}")


def _is_leaf(policy) -> bool:
    return isinstance(policy, str) or (isinstance(policy, tuple) and policy and isinstance(policy[0], str))


@contextmanager
def block_torch_functional(excludes=()):
    """Make torch.nn.functional.* raise inside the block (reference lines 40-62)."""
    saved = {}

    def make_stub(fname):
        def stub(*_a, **_k):
            raise RuntimeError(f"Function torch.nn.functional.{fname} is not allowed in this context.")
        return stub

    for fname in dir(F):
        if fname.startswith("_") or fname in excludes:
            continue
        obj = getattr(F, fname)
        if callable(obj):
            saved[fname] = obj
            setattr(F, fname, make_stub(fname))
    try:
        yield
    finally:
        for fname, obj in saved.items():
            setattr(F, fname, obj)


def initialize_models(model, model_new):
    if not torch.cuda.is_available():
        raise RuntimeError("verification needs a CUDA device: ModelNew has no CPU path")
    init = as_list(model.get_init_inputs())
    torch_model = model.Model(*init).eval().cuda()
    cuda_model = model_new.ModelNew(*init).eval().cuda()
    cuda_model.load_state_dict(torch_model.state_dict())
    return torch_model, cuda_model


def build_inputs(model):
    host = as_list(model.get_inputs())
    torch_inputs = map_tensors(host, lambda t: t.cuda())
    cuda_inputs = map_tensors(torch_inputs, lambda t: t.clone())
    return torch_inputs, cuda_inputs


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description="Check ModelNew against the eager Model.")
    add_workspace_args(parser)
    parser.add_argument("--checks", type=int, default=5, help="number of trials (reference: 5)")
    args = parser.parse_args(argv)
    model, model_new = load_task(args)
    policy = getattr(model, "OUTPUT_POLICY", None)
    torch_model, cuda_model = initialize_models(model, model_new)
    with torch.no_grad():
        for i in range(args.checks):
            torch_inputs, cuda_inputs = build_inputs(model)
            expected = torch_model(*torch_inputs)
            with block_torch_functional():
                actual = cuda_model(*cuda_inputs)
            metrics = check_equal(actual, expected, policy)
            detail = "; ".join(
                "exact" if m["policy"] == "exact" else "rel_l2=%.2e max_abs=%.2e" % (m["rel_l2"], m["max_abs"])
                for m in metrics)
            print(f"[PASS] check {i + 1}/{args.checks}  ({detail})")
    torch.cuda.synchronize()
    print("[PASS] verify success")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
