"""ctypes access to the C ABI (``include/cuda_agent_b200.h``).

Each wrapper takes torch CUDA tensors, checks nothing that the launcher itself
checks, passes raw device pointers and the current torch stream, and raises
``CabError`` on a non-zero status. This is how the GPU tests and ``bench.py``
reach the kernels without going through pybind.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libcuda_agent_b200.so"

# name -> (restype, argtypes); one entry per declaration in include/cuda_agent_b200.h
SIGNATURES = {
    "cab_status_string": (c_char_p, [c_int]),
    "cab_version": (c_int, []),
    "axpby_launcher": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p]),
    "gdn_decode_launcher": (c_int, [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_void_p]),
}


class CabError(RuntimeError):
    def __init__(self, op: str, status: int, text: str):
        super().__init__(f"{op} failed with status {status}: {text}")
        self.status = status


_lib = None


def lib() -> ctypes.CDLL:
    """Load the launcher library once; there is no fallback when it is absent."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing: run `python -m cuda_agent_b200.build`")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = handle
    return _lib


def status_string(status: int) -> str:
    return lib().cab_status_string(status).decode()


def _check(op: str, status: int) -> None:
    if status != 0:
        raise CabError(op, status, status_string(status))


def _stream() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def _p(t) -> int:
    if not t.is_cuda:
        raise ValueError("the C ABI takes device pointers; got a CPU tensor")
    if not t.is_contiguous():
        raise ValueError("the C ABI takes contiguous buffers")
    return t.data_ptr()


def axpby(out, a, b, alpha: float, config: int = 0) -> None:
    _check("axpby_launcher",
           lib().axpby_launcher(_p(out), _p(a), _p(b), alpha, a.numel(), config, _stream()))


def gdn_decode(state, out, q, k, v, g, beta, config: int = 0) -> None:
    """One decode step; `state` [B,Hv,128,128] fp32 is updated in place, `out` [B,Hv,128] fp32."""
    B, Hv = state.shape[0], state.shape[1]
    Hq = q.shape[1]
    _check("gdn_decode_launcher",
           lib().gdn_decode_launcher(_p(state), _p(out), _p(q), _p(k), _p(v), _p(g), _p(beta),
                                     B, Hq, Hv, config, _stream()))
