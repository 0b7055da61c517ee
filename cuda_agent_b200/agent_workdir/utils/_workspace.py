"""Locating the two halves of a task for the verification and profiling loops.

The reference loops run from the workspace directory and do
``from model import ...`` / ``from model_new import ModelNew``
(agent_workdir/utils/verification.py:8-9). This workspace serves several tasks,
so both loops accept

  --task DIR        directory holding ``model_new.py`` (default: current directory)
  --model-dir DIR   directory holding the eager ``model.py`` (default: --task)

and otherwise behave as the reference does: with no flags, ``model.py`` and
``model_new.py`` are taken from the current directory.
"""
from __future__ import annotations

import argparse
import importlib
import sys
from pathlib import Path

WORKDIR = Path(__file__).resolve().parent.parent


def add_workspace_args(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--task", type=str, default=".", help="directory with model_new.py")
    parser.add_argument("--model-dir", type=str, default=None,
                        help="directory with the eager model.py (default: --task)")


def load_task(args):
    """Import (model, model_new) according to --task / --model-dir."""
    task = Path(args.task).resolve()
    model_dir = Path(args.model_dir).resolve() if args.model_dir else task
    # cuda_extension.so sits in the workspace root; model_new.py imports it by name.
    for p in (str(WORKDIR), str(model_dir), str(task)):
        if p in sys.path:
            sys.path.remove(p)
        sys.path.insert(0, p)
    for name in ("model", "model_new"):
        sys.modules.pop(name, None)
    model = importlib.import_module("model")
    model_new = importlib.import_module("model_new")
    return model, model_new


def map_tensors(obj, fn):
    """Apply fn to every tensor in a nest of list / tuple / dict (lists come back as lists)."""
    import torch
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, (list, tuple)):
        return [map_tensors(x, fn) for x in obj]
    if isinstance(obj, dict):
        return {key: map_tensors(val, fn) for key, val in obj.items()}
    return obj


def as_list(x):
    return list(x) if isinstance(x, (list, tuple)) else [x]
