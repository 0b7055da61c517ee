"""Assemble a self-contained ``agent_workdir`` for one task.

The reference's loop works on ONE directory: it compiles every ``*.cu`` / ``*.cpp`` in the directory and in
``kernels/`` (agent_workdir/utils/compile.py:11-20), imports ``model.py`` and ``model_new.py`` from it
(agent_workdir/utils/verification.py:8-9) and is driven by ``cd`` alone. This package keeps several tasks in
one workspace; ``export`` writes the directory the reference's loop expects for one of them:

    python -m cuda_agent_b200.export_task <task> <dest>      # task: gdn | mla | moe | moe_ep
    cd <dest>
    TORCH_CUDA_ARCH_LIST=10.0a bash utils/compile.sh --torch-load
    python3 -m utils.verification
    python3 -m utils.profiling --iters 10

What goes in: ``binding.cpp``, ``binding_registry.h``, ``kernels/`` (all launchers: the tasks share them),
``utils/``, the public header (as ``include/cuda_agent_b200.h`` inside the directory, with the two relative
``#include`` lines adjusted), the task's eager ``model.py`` (from ``oracle/<task>/``), its ``model_new.py`` and
its hand-over text as ``SKILL.md`` (the reference's name for the description an agent reads,
agent_workdir/SKILL.md). The eager model's configuration is chosen by the environment variable the model
documents (``CAB_GDN_CONFIG`` and so on); ``export`` records the one it was given in ``TASK_CONFIG.env``.
"""
from __future__ import annotations

import argparse
import shutil
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
WORKDIR = PKG / "agent_workdir"

# task -> (oracle directory holding model.py, environment variable that picks the eager model's configuration)
TASKS = {
    "gdn": ("gdn", "CAB_GDN_CONFIG"),
    "mla": ("mla", "CAB_MLA_CONFIG"),
    "moe": ("moe", "CAB_MOE_CONFIG"),
    "moe_ep": ("moe", "CAB_MOE_CONFIG"),
}
# the smallest configuration of each eager model that the CUDA operator accepts
DEFAULT_CONFIG = {"gdn": 0, "mla": 1, "moe": 0, "moe_ep": 1}


def export(task: str, dest: Path, config: int | None = None) -> Path:
    if task not in TASKS:
        raise ValueError(f"unknown task {task!r}; one of {sorted(TASKS)}")
    dest = Path(dest)
    if dest.exists() and any(dest.iterdir()):
        raise FileExistsError(f"{dest} exists and is not empty")
    dest.mkdir(parents=True, exist_ok=True)
    oracle_dir, env_name = TASKS[task]
    for name in ("binding.cpp", "binding_registry.h"):
        shutil.copy2(WORKDIR / name, dest / name)
    shutil.copytree(WORKDIR / "kernels", dest / "kernels", ignore=shutil.ignore_patterns("__pycache__"))
    shutil.copytree(WORKDIR / "utils", dest / "utils", ignore=shutil.ignore_patterns("__pycache__"))
    (dest / "include").mkdir()
    shutil.copy2(ROOT / "include" / "cuda_agent_b200.h", dest / "include" / "cuda_agent_b200.h")
    # the kernels reach the header by a path relative to kernels/: three levels up in the package, one here
    for name in ("cab_common.cuh", "binding_common.h"):
        f = dest / "kernels" / name
        f.write_text(f.read_text().replace("../../../include/cuda_agent_b200.h", "../include/cuda_agent_b200.h"))
    shutil.copy2(ROOT / "oracle" / oracle_dir / "model.py", dest / "model.py")
    shutil.copy2(WORKDIR / "tasks" / task / "model_new.py", dest / "model_new.py")
    shutil.copy2(WORKDIR / "tasks" / task / "README.md", dest / "SKILL.md")
    cfg = DEFAULT_CONFIG[task] if config is None else config
    (dest / "TASK_CONFIG.env").write_text(f"{env_name}={cfg}\n")
    return dest


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Write a self-contained agent_workdir for one task.")
    ap.add_argument("task", choices=sorted(TASKS))
    ap.add_argument("dest", type=Path)
    ap.add_argument("--config", type=int, default=None, help="configuration of the eager model (default: the smallest)")
    args = ap.parse_args(argv)
    out = export(args.task, args.dest, args.config)
    env = (out / "TASK_CONFIG.env").read_text().strip()
    print(f"wrote {out}\n  cd {out}\n  TORCH_CUDA_ARCH_LIST=10.0a bash utils/compile.sh --torch-load\n"
          f"  {env} python3 -m utils.verification\n  {env} python3 -m utils.profiling --iters 10")
    return 0


if __name__ == "__main__":
    sys.exit(main())
