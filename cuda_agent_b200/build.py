"""In-tree build of the two shared objects this package ships.

* ``cuda_agent_b200/lib/libcuda_agent_b200.so`` - every ``kernels/*.cu`` file,
  compiled by nvcc for sm_100a only; exports the ``extern "C"`` launchers declared
  in ``include/cuda_agent_b200.h``. It depends on no torch library.
* ``cuda_agent_b200/agent_workdir/cuda_extension.so`` - ``binding.cpp`` plus every
  ``kernels/*_binding.cpp``, compiled by g++ against the torch headers and linked
  to the library above. This is the module ``model_new.py`` imports.

The reference workspace builds one ``cuda_extension.so`` from the same file
layout with ``torch.utils.cpp_extension.load`` (agent_workdir/utils/compile.py:42-50);
that route still works on this directory (``agent_workdir/utils/compile.py`` here
keeps it). This builder exists because the launcher library must be loadable
without torch, and because compiling only what changed keeps a kernel edit to a
few seconds.

Compile flags follow the reference (``-O3 -std=c++17`` for C++, ``-O3
--use_fast_math`` for CUDA, agent_workdir/utils/compile.py:48-49) plus the explicit
``-gencode arch=compute_100a,code=sm_100a -lineinfo``.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
WORKDIR = PKG / "agent_workdir"
KERNELS = WORKDIR / "kernels"
LIB_DIR = PKG / "lib"
OBJ_DIR = ROOT / "build" / "obj"
CAPI_LIB = LIB_DIR / "libcuda_agent_b200.so"
EXT_SO = WORKDIR / "cuda_extension.so"

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
CXX = os.environ.get("CXX") or shutil.which("g++") or "g++"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "--use_fast_math",
    "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wno-attributes"]


class BuildError(RuntimeError):
    pass


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError("command failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))


def _headers(src: Path) -> list[Path]:
    """Headers a source of this kind may include (CUDA sources never include the
    binding headers and the reverse), so that a kernel edit does not recompile
    the torch-heavy binding files."""
    public = list((ROOT / "include").glob("*.h"))
    if src.suffix == ".cu":
        return sorted(list(KERNELS.glob("*.cuh")) + public)
    return sorted(list(KERNELS.glob("*.h")) + list(WORKDIR.glob("*.h")) + public)


def _stamp(src: Path, flags: list[str]) -> str:
    """Content hash of a source, the headers it may include and its flags."""
    h = hashlib.sha256()
    for p in [src] + _headers(src):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _compile_one(src: Path, compiler: str, flags: list[str]) -> tuple[Path, bool]:
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    obj = OBJ_DIR / (src.name + ".o")
    stamp_file = OBJ_DIR / (src.name + ".stamp")
    stamp = _stamp(src, [compiler] + flags)
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj, False
    _run([compiler] + flags + ["-c", str(src), "-o", str(obj)])
    stamp_file.write_text(stamp)
    return obj, True


def kernel_sources() -> list[Path]:
    return sorted(KERNELS.glob("*.cu"))


def binding_sources() -> list[Path]:
    return [WORKDIR / "binding.cpp"] + sorted(KERNELS.glob("*_binding.cpp"))


def _nccl_paths() -> tuple[list[str], list[str]]:
    """Include and link flags for the NCCL that torch itself loads."""
    try:
        import nvidia.nccl as nccl_pkg  # type: ignore
        base = Path(list(nccl_pkg.__path__)[0])
    except Exception:
        return [], []
    inc, lib = base / "include", base / "lib"
    if not (inc / "nccl.h").exists():
        return [], []
    return ["-I", str(inc)], ["-L" + str(lib), "-l:libnccl.so.2", "-Wl,-rpath," + str(lib)]


def build_capi(verbose: bool = False) -> Path:
    """Compile every kernels/*.cu and link libcuda_agent_b200.so."""
    srcs = kernel_sources()
    if not srcs:
        raise BuildError("no kernels/*.cu found under %s" % KERNELS)
    nccl_inc, nccl_link = _nccl_paths()
    flags = NVCC_FLAGS + nccl_inc
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        results = list(pool.map(lambda s: _compile_one(s, NVCC, flags), srcs))
    objs = [o for o, _ in results]
    changed = any(c for _, c in results)
    if verbose:
        for (o, c), s in zip(results, srcs):
            print("[build] %-28s %s" % (s.name, "compiled" if c else "up to date"))
    if changed or not CAPI_LIB.exists():
        LIB_DIR.mkdir(parents=True, exist_ok=True)
        needs_nccl = any("nccl" in s.read_text() for s in srcs)
        _run([NVCC, "-shared", "-o", str(CAPI_LIB)] + [str(o) for o in objs]
             + ["-gencode", "arch=compute_100a,code=sm_100a"]
             + ([a for f in nccl_link for a in ("-Xlinker", f)] if needs_nccl else []))
    return CAPI_LIB


def build_extension(verbose: bool = False) -> Path:
    """Compile binding.cpp + kernels/*_binding.cpp and link cuda_extension.so."""
    import torch.utils.cpp_extension as cpp_ext

    if not CAPI_LIB.exists():
        build_capi(verbose)
    incs: list[str] = []
    for p in cpp_ext.include_paths() + ["/usr/local/cuda/include", sysconfig.get_paths()["include"]]:
        incs += ["-isystem", p]
    try:
        import pybind11
        incs += ["-isystem", pybind11.get_include()]
    except ImportError:
        pass
    import torch
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    flags = CXX_FLAGS + incs + ["-DTORCH_EXTENSION_NAME=cuda_extension", "-DTORCH_API_INCLUDE_EXTENSION_H",
                                "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi]
    srcs = binding_sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        results = list(pool.map(lambda s: _compile_one(s, CXX, flags), srcs))
    if verbose:
        for (o, c), s in zip(results, srcs):
            print("[build] %-28s %s" % (s.name, "compiled" if c else "up to date"))
    changed = any(c for _, c in results)
    if changed or not EXT_SO.exists() or EXT_SO.stat().st_mtime < CAPI_LIB.stat().st_mtime:
        torch_lib = cpp_ext.library_paths()[0]
        _run([CXX, "-shared", "-o", str(EXT_SO)] + [str(o) for o, _ in results]
             + ["-L" + str(LIB_DIR), "-lcuda_agent_b200", "-Wl,-rpath,$ORIGIN/../lib",
                "-L" + torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
                "-ltorch_python"])
    return EXT_SO


def build_all(verbose: bool = False) -> None:
    build_capi(verbose)
    build_extension(verbose)


if __name__ == "__main__":
    try:
        build_all(verbose=True)
    except BuildError as exc:
        print(exc, file=sys.stderr)
        sys.exit(1)
    print("[build] ok: %s, %s" % (CAPI_LIB, EXT_SO))
