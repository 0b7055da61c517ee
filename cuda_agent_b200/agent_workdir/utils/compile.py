#!/usr/bin/env python3
"""Build ``cuda_extension.so`` for this workspace.

``python3 -m utils.compile`` from the workspace directory, as in the reference
(agent_workdir/utils/compile.py:66-71; wrapped by utils/compile.sh). Two routes:

* default: the package's incremental builder (``cuda_agent_b200/build.py``):
  nvcc for ``kernels/*.cu`` into ``libcuda_agent_b200.so``, g++ for ``binding.cpp``
  and ``kernels/*_binding.cpp`` into ``./cuda_extension.so``;
* ``--torch-load``: the reference's route, one ``torch.utils.cpp_extension.load``
  over ``*.cu`` and ``*.cpp`` in ``.`` and ``kernels/`` with the reference's flags
  (agent_workdir/utils/compile.py:11-20, :42-50). The target architecture then
  comes from ``TORCH_CUDA_ARCH_LIST`` (use ``10.0a``), as it does there.

Exit status 0 on success, 1 on failure, and the same final line
``Compile success: cuda_extension.so``.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys
from pathlib import Path

WORKDIR = Path(__file__).resolve().parent.parent


def find_sources(workdir: Path) -> list[str]:
    found: set[str] = set()
    for folder in (workdir, workdir / "kernels"):
        if folder.is_dir():
            for pattern in ("*.cu", "*.cpp"):
                found.update(str(p) for p in folder.glob(pattern))
    return sorted(found)


def compile_with_torch_load(workdir: Path) -> int:
    import torch.utils.cpp_extension as cpp_ext

    sources = find_sources(workdir)
    if not sources:
        print("Error: no source files found (*.cu, *.cpp in root or kernels/)")
        return 1
    print(f"Compiling {len(sources)} files: {', '.join(os.path.relpath(s, workdir) for s in sources)}")
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    build_dir = workdir / "build" / "forced_compile"
    shutil.rmtree(build_dir, ignore_errors=True)
    build_dir.mkdir(parents=True)
    target = workdir / "cuda_extension.so"
    target.unlink(missing_ok=True)
    try:
        cpp_ext.load(name="cuda_extension", sources=sources, build_directory=str(build_dir),
                     verbose=False, with_cuda=True, extra_cflags=["-O3", "-std=c++17"],
                     extra_cuda_cflags=["-O3", "--use_fast_math", "-lineinfo"])
    except Exception as exc:  # the reference prints and returns 1 on any build error
        print("Compilation failed.")
        print(str(exc))
        return 1
    built = build_dir / "cuda_extension.so"
    if not built.exists():
        print("Compilation finished but cuda_extension.so was not generated.")
        return 1
    shutil.copy2(built, target)
    print(f"Compile success: {target.name}")
    return 0


def compile_incremental() -> int:
    sys.path.insert(0, str(WORKDIR.parent.parent))
    from cuda_agent_b200 import build as pkg_build

    try:
        pkg_build.build_all(verbose=True)
    except pkg_build.BuildError as exc:
        print("Compilation failed.")
        print(str(exc))
        return 1
    print(f"Compile success: {pkg_build.EXT_SO.name}")
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description="Compile the workspace's CUDA extension.")
    parser.add_argument("--torch-load", action="store_true",
                        help="single torch.utils.cpp_extension.load build, as the reference does")
    args = parser.parse_args(argv)
    # a workspace exported for one task stands alone (no package around it): the reference's route is the only one
    standalone = not (WORKDIR.parent / "build.py").exists()
    if args.torch_load or standalone:
        return compile_with_torch_load(Path.cwd())
    return compile_incremental()


if __name__ == "__main__":
    sys.exit(main())
