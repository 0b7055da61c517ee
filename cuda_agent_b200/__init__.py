"""B200 (sm_100a) operators behind the CUDA-Agent ``agent_workdir`` operator API.

What is here:

* ``agent_workdir/`` - a workspace in the reference's shape: ``binding.cpp``,
  ``binding_registry.h``, ``kernels/*.cu`` (+ ``*_binding.cpp``), ``utils/`` with the
  compile / verification / profiling loops, and one ``tasks/<name>/model_new.py``
  per operator path;
* ``capi`` - ctypes access to ``lib/libcuda_agent_b200.so``, the C ABI declared in
  ``include/cuda_agent_b200.h``;
* ``build`` - the in-tree builder of both shared objects.

There is no CPU implementation of any operator in this package: loading fails
with an ImportError when the shared objects have not been built, and every
operator raises when handed a non-CUDA tensor.
"""
from pathlib import Path

__version__ = "0.1.0"

PACKAGE_DIR = Path(__file__).resolve().parent
WORKDIR = PACKAGE_DIR / "agent_workdir"


def load_extension():
    """Import and return the ``cuda_extension`` pybind module of the workspace."""
    import importlib
    import sys

    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    so = WORKDIR / "cuda_extension.so"
    if not so.exists():
        raise ImportError(
            f"{so} is missing: build it with `python -m cuda_agent_b200.build` "
            "(there is no fallback implementation)")
    if str(WORKDIR) not in sys.path:
        sys.path.insert(0, str(WORKDIR))
    return importlib.import_module("cuda_extension")
