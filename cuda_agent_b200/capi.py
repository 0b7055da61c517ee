"""ctypes access to the C ABI (``include/cuda_agent_b200.h``).

Each wrapper takes torch CUDA tensors, checks nothing that the launcher itself
checks, passes raw device pointers and the current torch stream, and raises
``CabError`` on a non-zero status. This is how the GPU tests and ``bench.py``
reach the kernels without going through pybind.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libcuda_agent_b200.so"

# name -> (restype, argtypes); one entry per declaration in include/cuda_agent_b200.h
SIGNATURES = {
    "cab_status_string": (c_char_p, [c_int]),
    "cab_version": (c_int, []),
    "cab_wait_selftest": (c_int, [c_void_p, ctypes.c_longlong, c_int, c_void_p]),
    "axpby_launcher": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p]),
    "gdn_decode_launcher": (c_int, [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_void_p]),
    "moe_router_logits_launcher": (c_int, [c_void_p] * 3 + [c_int] * 4 + [c_void_p]),
    "moe_route_softmax_topk_launcher": (c_int, [c_void_p] * 3 + [c_int] * 4 + [c_void_p]),
    "moe_route_sigmoid_group_topk_launcher": (c_int, [c_void_p] * 4 + [c_int] * 5 + [c_float, c_int, c_void_p]),
    "moe_permute_scratch_bytes": (c_size_t, [c_int, c_int, c_int]),
    "moe_permute_max_tiles": (c_int, [c_int, c_int, c_int]),
    "moe_permute_launcher": (c_int, [c_void_p, c_int, c_int, c_int] + [c_void_p] * 8 + [c_int, c_void_p, c_int, c_void_p]),
    "moe_quant_dispatch_launcher": (c_int, [c_void_p] * 4 + [c_int] * 5 + [c_void_p]),
    "moe_quant_rows_launcher": (c_int, [c_void_p] * 4 + [c_int] * 4 + [c_void_p]),
    "moe_scatter_rows_launcher": (c_int, [c_void_p] * 5 + [c_int] * 4 + [c_void_p]),
    "moe_gather_rows_launcher": (c_int, [c_void_p] * 3 + [c_int] * 3 + [c_void_p]),
    "moe_tiles_from_counts_launcher": (c_int, [c_void_p, c_int] + [c_void_p] * 4 + [c_int, c_int, c_void_p]),
    "moe_combine_launcher": (c_int, [c_void_p] * 5 + [c_int] * 4 + [c_void_p]),
    "mla_sparse_decode_scratch_bytes": (c_size_t, [c_int, c_int, c_int]),
    "mla_sparse_decode_launcher": (c_int, [c_void_p] * 5 + [c_int] * 4 + [c_float, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "mla_sparse_decode_multi_launcher": (c_int, [c_void_p] * 5 + [c_int] * 5 + [c_float, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "mla_sparse_decode_noalloc_launcher": (c_int, [c_void_p] * 5 + [c_int] * 4 + [c_float, c_int, c_void_p, c_int, c_void_p]),
    "mla_gather_rows_launcher": (c_int, [c_void_p] * 4 + [c_int] * 4 + [c_void_p]),
    "moe_grouped_gemm_fp8_launcher": (c_int, [c_int] + [c_void_p] * 8 + [c_int] * 6 + [c_void_p, c_int, c_void_p]),
    "moe_ep_peer_buffer_bytes": (c_size_t, [c_int] * 4),
    "moe_ep_peer_create": (c_int, [c_void_p] + [c_int] * 6),
    "moe_ep_peer_export": (c_int, [c_void_p, c_void_p]),
    "moe_ep_peer_connect_ipc": (c_int, [c_void_p, c_void_p]),
    "moe_ep_peer_connect_local": (c_int, [c_void_p, c_void_p]),
    "moe_ep_peer_destroy": (c_int, [c_void_p]),
    "moe_ep_peer_dispatch_launcher": (c_int, [c_void_p] * 4 + [c_int, c_int, c_void_p]),
    "moe_ep_peer_receive_launcher": (c_int, [c_void_p, c_int, c_void_p]),
    "moe_ep_peer_gather_launcher": (c_int, [c_void_p] * 4 + [c_int, c_int, c_void_p]),
    "moe_ep_peer_return_launcher": (c_int, [c_void_p] * 3 + [c_int, c_void_p]),
    "moe_ep_peer_combine_launcher": (c_int, [c_void_p] * 3 + [c_int, c_int, c_void_p]),
    "moe_ep_peer_workspace_bytes": (c_size_t, [c_void_p, c_void_p]),
    "moe_ep_peer_layer_launcher": (c_int, [c_void_p] * 3 + [c_int, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "moe_ep_peer_read_status": (c_int, [c_void_p] * 4),
    "moe_ep_peer_debug_read": (c_int, [c_void_p, c_int, c_size_t, c_void_p, c_size_t]),
}


class MoeEpLayerArgs(ctypes.Structure):
    """`cab_moe_ep_layer_args` of the header, field for field."""
    _fields_ = [(n, c_void_p) for n in ("router_w", "router_bias", "w13_q", "w13_s", "w2_q", "w2_s", "shared_w13_q",
                                        "shared_w13_s", "shared_w2_q", "shared_w2_s")] + \
               [("E", c_int), ("I", c_int), ("routing", c_int), ("n_group", c_int), ("topk_group", c_int),
                ("scaling", c_float), ("entry_cap", c_int), ("gemm_ctas", c_int)]


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


def wait_selftest(status, limit_cycles: int, withhold: bool) -> None:
    """Runs the bounded-wait self-test kernel; `status` (int32 [1], CUDA) receives 0 or the give-up code 901."""
    _check("cab_wait_selftest",
           lib().cab_wait_selftest(_p(status), int(limit_cycles), int(bool(withhold)), _stream()))


def axpby(out, a, b, alpha: float, config: int = 0) -> None:
    _check("axpby_launcher",
           lib().axpby_launcher(_p(out), _p(a), _p(b), alpha, a.numel(), config, _stream()))


GDN_REVERSE = 16


def gdn_loop_config(step: int, config: int = 0) -> int:
    """`config` for step `step` of a decode loop on one state: the reverse-walk bit on odd steps, so that every
    step starts on the rows the previous one wrote last (still in L2). The result of a step does not depend on
    the bit."""
    return (config & 15) | (GDN_REVERSE if step & 1 else 0)


def gdn_decode(state, out, q, k, v, g, beta, config: int = 0) -> None:
    """One decode step; `state` [B,Hv,128,128] fp32 is updated in place, `out` [B,Hv,128] fp32."""
    B, Hv = state.shape[0], state.shape[1]
    Hq = q.shape[1]
    _check("gdn_decode_launcher",
           lib().gdn_decode_launcher(_p(state), _p(out), _p(q), _p(k), _p(v), _p(g), _p(beta),
                                     B, Hq, Hv, config, _stream()))


# ----------------------------------------------------------------------------- MoE stages
def _opt(t):
    return None if t is None else _p(t)


def moe_router_logits(logits, x, wr, config: int = 0) -> None:
    T, H = x.shape
    _check("moe_router_logits_launcher",
           lib().moe_router_logits_launcher(_p(logits), _p(x), _p(wr), T, H, wr.shape[0], config, _stream()))


def moe_route_softmax_topk(topk_idx, topk_w, logits, config: int = 0) -> None:
    T, E = logits.shape
    _check("moe_route_softmax_topk_launcher",
           lib().moe_route_softmax_topk_launcher(_p(topk_idx), _p(topk_w), _p(logits), T, E,
                                                 topk_idx.shape[1], config, _stream()))


def moe_route_sigmoid_group_topk(topk_idx, topk_w, logits, bias, n_group, topk_group, scale=1.0,
                                 config: int = 0) -> None:
    T, E = logits.shape
    _check("moe_route_sigmoid_group_topk_launcher",
           lib().moe_route_sigmoid_group_topk_launcher(_p(topk_idx), _p(topk_w), _p(logits), _p(bias), T, E,
                                                       topk_idx.shape[1], n_group, topk_group, scale,
                                                       config, _stream()))


def moe_permute(topk_idx, E: int, config: int = 0):
    """Allocates and returns the permutation tables for topk_idx [T, k] (int32, CUDA).
    config bit 0: an id of -1 marks an empty slot and is skipped without raising the flag."""
    import torch
    T, k = topk_idx.shape
    dev = topk_idx.device
    i32 = dict(dtype=torch.int32, device=dev)
    max_tiles = lib().moe_permute_max_tiles(T, k, E)
    out = dict(counts=torch.empty(E, **i32), offsets=torch.empty(E + 1, **i32),
               pad_offsets=torch.empty(E + 1, **i32), perm=torch.empty(T * k, **i32),
               inv_perm=torch.empty(T * k, **i32), dst_row=torch.empty(T * k, **i32),
               tile_expert=torch.empty(max_tiles, **i32), num_tiles=torch.empty(1, **i32),
               max_tiles=max_tiles)
    scratch = torch.empty(lib().moe_permute_scratch_bytes(T, k, E), dtype=torch.uint8, device=dev)
    _check("moe_permute_launcher",
           lib().moe_permute_launcher(_p(topk_idx), T, k, E, _p(out["counts"]), _p(out["offsets"]),
                                      _p(out["pad_offsets"]), _p(out["perm"]), _p(out["inv_perm"]),
                                      _p(out["dst_row"]), _p(out["tile_expert"]), _p(out["num_tiles"]),
                                      max_tiles, _p(scratch), config, _stream()))
    out["scratch"] = scratch
    return out


def moe_quant_dispatch(a_q, scales_t, x, dst_row, k: int, config: int = 0) -> None:
    T, H = x.shape
    _check("moe_quant_dispatch_launcher",
           lib().moe_quant_dispatch_launcher(_p(a_q), _p(scales_t), _p(x), _opt(dst_row), T, H, k,
                                             scales_t.shape[1], config, _stream()))


def moe_combine(out, y, dst_row, weights, extra=None, config: int = 0) -> None:
    T, H = out.shape
    _check("moe_combine_launcher",
           lib().moe_combine_launcher(_p(out), _p(y), _p(dst_row), _p(weights), _opt(extra), T, H,
                                      weights.shape[1], config, _stream()))


def moe_grouped_gemm_fp8(mode, out, out_scales_t, a_q, a_scales_t, w_q, w_scales, tile_expert, num_tiles,
                         max_m_tiles, status=None, config: int = 0) -> None:
    """mode 0: gate/up + SwiGLU + re-quantise; mode 1: down projection to bf16 (see the header)."""
    rows_cap, K = a_q.shape
    E = w_q.shape[0]
    N = out.shape[1]
    _check("moe_grouped_gemm_fp8_launcher",
           lib().moe_grouped_gemm_fp8_launcher(mode, _p(out), _opt(out_scales_t), _p(a_q), _p(a_scales_t),
                                               _p(w_q), _p(w_scales), _opt(tile_expert), _opt(num_tiles),
                                               max_m_tiles, rows_cap, a_scales_t.shape[1], E, N, K,
                                               _opt(status), config, _stream()))


# ----------------------------------------------------------------------------- sparse MLA decode
def mla_sparse_decode(out, q, kv, seq_len, idx, softmax_scale: float, nsplit: int = 1, scratch=None, status=None,
                      config: int = 0) -> None:
    B, _, Hh, _ = q.shape
    S, topk = kv.shape[1], idx.shape[-1]
    _check("mla_sparse_decode_launcher",
           lib().mla_sparse_decode_launcher(_p(out), _p(q), _p(kv), _p(seq_len), _p(idx), B, Hh, S, topk,
                                            softmax_scale, nsplit, _opt(scratch), _opt(status), config, _stream()))


def mla_sparse_decode_multi(out, q, kv, seq_len, idx, softmax_scale: float, nsplit: int = 1, scratch=None,
                            status=None, config: int = 0) -> None:
    """q [B, Sq, Hh, 576], seq_len [B, Sq], idx [B, Sq, topk], out [B, Sq, Hh, 512]: Sq query tokens per sequence."""
    B, Sq, Hh, _ = q.shape
    S, topk = kv.shape[1], idx.shape[-1]
    _check("mla_sparse_decode_multi_launcher",
           lib().mla_sparse_decode_multi_launcher(_p(out), _p(q), _p(kv), _p(seq_len), _p(idx), B, Sq, Hh, S, topk,
                                                  softmax_scale, nsplit, _opt(scratch), _opt(status), config,
                                                  _stream()))


def mla_scratch_bytes(B: int, Hh: int, nsplit: int) -> int:
    return lib().mla_sparse_decode_scratch_bytes(B, Hh, nsplit)


def mla_gather_rows(rows, kv, seq_len, idx, config: int = 0) -> None:
    B, S, _ = kv.shape
    _check("mla_gather_rows_launcher",
           lib().mla_gather_rows_launcher(_p(rows), _p(kv), _p(seq_len), _p(idx), B, S, idx.shape[-1], config,
                                          _stream()))


MLA_STATIC_SCRATCH_BYTES = 16 * 1024 * 1024


def mla_sparse_decode_noalloc(out, q, kv, seq_len, idx, softmax_scale: float, nsplit: int, status=None,
                              config: int = 0) -> None:
    """Split decode whose partials live in the library's fixed device array: nothing is allocated.

    For hosts that cannot hand over scratch memory (their allocator is closed while serving, or their
    operator interface has no workspace argument). Raises CabError(status 4) when
    B * nsplit * Hh * 2056 bytes exceed MLA_STATIC_SCRATCH_BYTES. Calls on one GPU share the array."""
    B, _, Hh, _ = q.shape
    S, topk = kv.shape[1], idx.shape[-1]
    _check("mla_sparse_decode_noalloc_launcher",
           lib().mla_sparse_decode_noalloc_launcher(_p(out), _p(q), _p(kv), _p(seq_len), _p(idx), B, Hh, S, topk,
                                                    softmax_scale, nsplit, _opt(status), config, _stream()))


# ----------------------------------------------------------------------------- expert-parallel row movement
def moe_quant_rows(rows_q, scales, x, dst_row, k: int) -> None:
    T, H = x.shape
    _check("moe_quant_rows_launcher",
           lib().moe_quant_rows_launcher(_p(rows_q), _p(scales), _p(x), _opt(dst_row), T, H, k, 0, _stream()))


def moe_scatter_rows(a_q, scales_t, rows, scales, dst_row) -> None:
    n, H = rows.shape
    _check("moe_scatter_rows_launcher",
           lib().moe_scatter_rows_launcher(_p(a_q), _p(scales_t), _p(rows), _p(scales), _p(dst_row), n, H,
                                           scales_t.shape[1], 0, _stream()))


def moe_gather_rows(out, y, src_row) -> None:
    n, H = out.shape
    _check("moe_gather_rows_launcher", lib().moe_gather_rows_launcher(_p(out), _p(y), _p(src_row), n, H, 0, _stream()))


def moe_tiles_from_counts(counts, offsets, pad_offsets, tile_expert, num_tiles) -> None:
    _check("moe_tiles_from_counts_launcher",
           lib().moe_tiles_from_counts_launcher(_p(counts), counts.numel(), _p(offsets), _p(pad_offsets),
                                                _p(tile_expert), _p(num_tiles), tile_expert.numel(), 0, _stream()))
