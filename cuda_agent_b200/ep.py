"""Expert-parallel MoE layer: one process per GPU, experts in contiguous blocks of E/N per rank.

Data path of one layer call on rank r (T local tokens, k experts per token):

  route            logits, top-k -> idx [T,k] (global expert ids), weights [T,k]          (kernels)
  permute          stable sort of the T*k entries by expert = by destination rank, then by
                   that rank's local expert                                               (kernels)
  quant_rows       1x128 e4m3 rows + row-major scales, written in sorted order            (kernel)
  counts exchange  all-to-all of the [N, E/N] population matrix                           (NCCL)
  dispatch         all-to-all of rows and scales with per-rank split sizes                (NCCL)
  expert_ffn       scatter into the padded row space, grouped GEMM gate/up (+SwiGLU+
                   re-quantise), grouped GEMM down, gather back into arrival order        (kernels)
  return           all-to-all of the bf16 result rows, split sizes reversed               (NCCL)
  combine          weighted sum per token in slot order (+ shared expert)                 (kernel)

That is `ep_moe_forward(..., dedup=False)`: an entry travels once per (token, slot). The default is the
merged form (`_ep_dedup`; on one rank it still saves the copy of the results back into arrival order): a token travels ONCE to every rank that holds at least
one of its experts (with group-limited routing at most `topk_group` ranks instead of k entries), together
with a side band of k (local expert, weight) slots; the receiving rank expands the copies into its padded
row space, runs the grouped GEMMs, forms the weighted sum of each copy's entries in fp32 and returns ONE
bf16 row per copy; the source adds the partial rows of a token (+ shared expert). Bytes on the wire drop by
the ratio entries / copies (2 x for 8 experts over 4 ranks). The split sizes are needed on the host, so
the population exchange ends in a device-to-host copy per call.

The bookkeeping (`ExchangePlan`) is integer tensor arithmetic that runs on any device; the compute is
behind an `ops` object so that the same schedule runs over NCCL with the CUDA kernels (`CudaOps`) and,
in the CPU tests, over gloo with a stand-in. `CudaOps` has no CPU path.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def _excl_cumsum(t: torch.Tensor, dim: int = 0) -> torch.Tensor:
    return torch.cumsum(t, dim) - t


@dataclass
class ExchangePlan:
    """Where every entry goes and where every received entry lands.

    send_splits[d]   entries this rank sends to rank d (sorted entries are contiguous per rank)
    recv_splits[s]   entries arriving from rank s (arrival order: by source rank, then local expert)
    local_counts[e]  population of local expert e over all sources
    dst_row[i]       row of arrival i in the padded row space (every expert starts at a multiple of 128)
    rows_cap         rows of that space (a multiple of 128)
    """
    send_splits: list
    recv_splits: list
    local_counts: torch.Tensor
    dst_row: torch.Tensor
    rows_cap: int

    @staticmethod
    def build(counts: torch.Tensor, world: int, group=None, tile: int = 128) -> "ExchangePlan":
        """counts: int32/int64 [E] entries of this rank per GLOBAL expert."""
        E = counts.numel()
        assert E % world == 0, "experts must divide evenly over the ranks"
        e_local = E // world
        send_mat = counts.reshape(world, e_local).to(torch.int64).contiguous()
        recv_mat = torch.empty_like(send_mat)
        if world > 1:
            dist.all_to_all_single(recv_mat, send_mat, group=group)
        else:
            recv_mat.copy_(send_mat)
        return ExchangePlan.from_matrices(send_mat, recv_mat, tile)

    @staticmethod
    def from_matrices(send_mat: torch.Tensor, recv_mat: torch.Tensor, tile: int = 128) -> "ExchangePlan":
        """send_mat [N, E/N]: my entries per (destination, its local expert); recv_mat [N, E/N]: entries
        per (source, my local expert)."""
        local_counts = recv_mat.sum(0)
        padded = (local_counts + tile - 1) // tile * tile
        pad_offsets = _excl_cumsum(padded)
        within = _excl_cumsum(recv_mat, 0)                         # rows of expert e that earlier sources fill
        block_dst = (pad_offsets[None, :] + within).reshape(-1)    # arrival blocks: source major, expert minor
        block_cnt = recv_mat.reshape(-1)
        block_start = _excl_cumsum(block_cnt)
        n_recv = int(block_cnt.sum())                              # host sync: the split sizes are host data
        dst_row = torch.repeat_interleave(block_dst - block_start, block_cnt, output_size=n_recv) \
            + torch.arange(n_recv, device=recv_mat.device)
        return ExchangePlan(send_splits=send_mat.sum(1).tolist(), recv_splits=recv_mat.sum(1).tolist(),
                            local_counts=local_counts.to(torch.int32), dst_row=dst_row.to(torch.int32),
                            rows_cap=max(int(padded.sum()), tile))


def _all_to_all_rows(send: torch.Tensor, send_splits, recv_splits, world: int, group=None) -> torch.Tensor:
    """Exchange of row blocks; rows are moved as bytes so that every backend accepts the dtype."""
    row_bytes = send.shape[1] * send.element_size()
    send_b = send.contiguous().view(torch.uint8).reshape(-1, row_bytes)
    recv_b = torch.empty(sum(recv_splits), row_bytes, dtype=torch.uint8, device=send.device)
    if world > 1:
        dist.all_to_all_single(recv_b, send_b, output_split_sizes=list(recv_splits),
                               input_split_sizes=list(send_splits), group=group)
    else:
        recv_b.copy_(send_b)
    return recv_b.view(send.dtype).reshape(-1, send.shape[1])


def _count(values: torch.Tensor, bins: int) -> torch.Tensor:
    """Occurrences of 0..bins-1 in `values` (int64), without the device-to-host copy torch.bincount makes."""
    return torch.zeros(bins, dtype=torch.int64, device=values.device).scatter_add_(0, values, torch.ones_like(values))


def _all_to_all_counts(n_send: torch.Tensor, world: int, group=None) -> torch.Tensor:
    n_recv = torch.empty_like(n_send)
    if world > 1:
        dist.all_to_all_single(n_recv, n_send, group=group)
    else:
        n_recv.copy_(n_send)
    return n_recv


def _ep_dedup(x: torch.Tensor, ops, world: int, group=None) -> torch.Tensor:
    """One copy of a token per destination rank; one partial result row per copy on the way back."""
    dev, T, H = x.device, x.shape[0], x.shape[1]
    nb = H // 128
    idx, w = ops.route(x)                                           # [T, k]
    k, e_local = idx.shape[1], ops.e_local
    begin = getattr(ops, "shared_expert_begin", None)
    pending = begin(x) if begin else None
    # ---- copies: (destination rank, token) pairs in that order
    dest = torch.div(idx, e_local, rounding_mode="floor").long()   # [T, k]
    has = torch.zeros(T, world, dtype=torch.bool, device=dev).scatter_(1, dest, True)
    has_t = has.t().contiguous().reshape(-1)                        # rank major, token minor
    pos = torch.cumsum(has_t.to(torch.int64), 0) - 1
    copy_pos = torch.where(has_t, pos, torch.full_like(pos, -1)).reshape(world, T).t().contiguous()   # [T, N]
    # per destination: copies and entries; the entry totals let the receiver size its row space without a
    # second device-to-host copy
    n_send = torch.stack([has.sum(0).to(torch.int64),
                          _count(dest.reshape(-1), world)], dim=1).contiguous()                      # [N, 2]
    n_recv = _all_to_all_counts(n_send, world, group)
    send_host, recv_host = torch.stack([n_send, n_recv]).tolist()   # the one host sync of the call
    send_splits, recv_splits = [c for c, _ in send_host], [c for c, _ in recv_host]
    n_copies, n_entries = sum(send_splits), sum(e for _, e in recv_host)
    # ---- side band of a copy: its scales, then k slots of (weight, expert local to the destination or -1)
    entry_copy = torch.gather(copy_pos, 1, dest)                    # [T, k] copy that carries entry (t, slot)
    slot = torch.arange(k, device=dev).expand(T, k)
    meta_e = torch.full((n_copies, k), -1, dtype=torch.int32, device=dev)
    meta_w = torch.zeros(n_copies, k, dtype=torch.float32, device=dev)
    meta_e[entry_copy, slot] = (idx.long() - dest * e_local).to(torch.int32)
    meta_w[entry_copy, slot] = w.float()
    copy_pos32 = copy_pos.to(torch.int32)
    rows, scales = ops.quant_copies(x, copy_pos32, n_copies)
    side = torch.cat([scales, meta_w, meta_e.view(torch.float32)], dim=1).contiguous()
    recv_rows = _all_to_all_rows(rows, send_splits, recv_splits, world, group)
    recv_side = _all_to_all_rows(side, send_splits, recv_splits, world, group)
    R = recv_rows.shape[0]
    r_scales = recv_side[:, :nb].contiguous()
    r_w = recv_side[:, nb:nb + k].contiguous()
    r_e = recv_side[:, nb + k:].contiguous().view(torch.int32)
    # ---- entries of the received copies, sorted by local expert (stable: arrival order, then slot),
    #      every expert's rows starting at a multiple of 128
    key = r_e.reshape(-1).long()
    key = torch.where(key >= 0, key, torch.full_like(key, e_local))
    order = torch.argsort(key, stable=True)
    local_counts = _count(key, e_local + 1)[:e_local]
    padded = (local_counts + 127) // 128 * 128
    # rows of the padded space: at most 127 rows of padding per expert (the tile table on the device knows
    # the exact extent; rows past it are never touched by a tile)
    cap = max((n_entries + e_local * 127 + 127) // 128 * 128, 128)
    live = order[:n_entries]
    live_e = key[live]
    dst = _excl_cumsum(padded)[live_e] + torch.arange(n_entries, device=dev) - _excl_cumsum(local_counts)[live_e]
    entry_row = torch.full((R * k,), -1, dtype=torch.int32, device=dev)
    entry_row[live] = dst.to(torch.int32)
    src_copy = torch.full((cap,), -1, dtype=torch.int32, device=dev)
    src_copy[dst] = torch.div(live, k, rounding_mode="floor").to(torch.int32)
    y = ops.expert_ffn_entries(recv_rows, r_scales, src_copy, local_counts.to(torch.int32), cap)   # [cap, H] bf16
    partial = ops.combine(y, entry_row, r_w, None)                  # [R, H]: sum_j w_j y_j of each copy, fp32 -> bf16
    back = _all_to_all_rows(partial, recv_splits, send_splits, world, group)
    shared = ops.shared_expert_end(pending) if begin else ops.shared_expert(x)
    return ops.combine(back, copy_pos32.reshape(-1), has.to(torch.float32), shared)


def ep_moe_forward(x: torch.Tensor, ops, world: int, group=None, micro_batches: int = 1, dedup=None) -> torch.Tensor:
    """One layer call on this rank; `ops` supplies the compute (see CudaOps for the contract).

    dedup (the default without micro-batching) sends a token once per destination rank, see the module
    text; micro-batching applies to the per-entry form only.

    With micro_batches = 2 the local tokens are processed as two halves on two CUDA streams, issued in
    an interleaved order: the dispatch of the second half travels while the experts work on the first,
    and the first half's results travel back while the experts work on the second. The result does not
    depend on the split (every token is computed independently of its neighbours)."""
    if dedup is None:
        dedup = micro_batches <= 1
    if dedup:
        return _ep_dedup(x, ops, world, group)
    if micro_batches <= 1 or x.shape[0] < 2 * micro_batches:
        return _ep_pipeline([x], ops, world, group)[0]
    bounds = [x.shape[0] * i // micro_batches for i in range(micro_batches + 1)]
    parts = [x[bounds[i]:bounds[i + 1]] for i in range(micro_batches)]
    return torch.cat(_ep_pipeline(parts, ops, world, group), dim=0)


_STREAMS = {}


def _part_streams(device, n):
    key = (device.index, n)
    if key not in _STREAMS:
        _STREAMS[key] = [torch.cuda.Stream(device=device) for _ in range(n)]
    return _STREAMS[key]


class _NoStream:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def _ep_pipeline(parts, ops, world: int, group=None):
    """The layer schedule for each part, stage by stage across parts (part i on its own stream when
    the tensors live on a GPU), so that exchanges of one part overlap the compute of another."""
    n = len(parts)
    on_gpu = parts[0].is_cuda and n > 1
    if on_gpu:
        cur = torch.cuda.current_stream(parts[0].device)
        streams = _part_streams(parts[0].device, n)
        for st in streams:
            st.wait_stream(cur)
    ctx = (lambda i: torch.cuda.stream(streams[i])) if on_gpu else (lambda i: _NoStream())
    begin = getattr(ops, "shared_expert_begin", None)
    st = [dict() for _ in range(n)]
    for i, x in enumerate(parts):                      # local routing, sorting, quantisation
        with ctx(i):
            s = st[i]
            s["idx"], s["w"] = ops.route(x)
            s["counts"], s["inv_perm"] = ops.permute(s["idx"])
            s["rows"], s["scales"] = ops.quant_rows(x, s["inv_perm"])
            # the shared expert depends on nothing that is exchanged: start it now on a side stream
            s["pending"] = begin(x) if begin else None
    for i in range(n):                                 # population exchange (host sync) and dispatch
        with ctx(i):
            s = st[i]
            s["plan"] = ExchangePlan.build(s["counts"], world, group)
            p = s["plan"]
            s["recv_rows"] = _all_to_all_rows(s["rows"], p.send_splits, p.recv_splits, world, group)
            s["recv_scales"] = _all_to_all_rows(s["scales"], p.send_splits, p.recv_splits, world, group)
    for i in range(n):                                 # experts, then the way back
        with ctx(i):
            s = st[i]
            p = s["plan"]
            y_recv = ops.expert_ffn(s["recv_rows"], s["recv_scales"], p)     # bf16 [n_recv, H], arrival order
            s["y_back"] = _all_to_all_rows(y_recv, p.recv_splits, p.send_splits, world, group)
    outs = []
    for i, x in enumerate(parts):                      # combine
        with ctx(i):
            s = st[i]
            shared = ops.shared_expert_end(s["pending"]) if begin else ops.shared_expert(x)
            outs.append(ops.combine(s["y_back"], s["inv_perm"], s["w"], shared))
    if on_gpu:
        for i, stream in enumerate(streams):
            cur.wait_stream(stream)
            outs[i].record_stream(cur)
    return outs


class CudaOps:
    """The compute steps on this rank's GPU, through the C ABI. Weights are this rank's expert block."""

    def __init__(self, router_w, router_bias, w13_q, w13_s, w2_q, w2_s, shared=None, k=8, routing=1, n_group=8,
                 topk_group=4, scaling=1.0, num_experts=None, gemm_ctas=0):
        from . import capi
        self.capi = capi
        capi.lib()
        self.router_w, self.router_bias = router_w, router_bias
        self.w13_q, self.w13_s, self.w2_q, self.w2_s = w13_q.view(torch.uint8), w13_s, w2_q.view(torch.uint8), w2_s
        self.shared = None if shared is None else tuple(
            t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t for t in shared)
        self.k, self.routing, self.n_group, self.topk_group, self.scaling = k, routing, n_group, topk_group, scaling
        self.E = num_experts if num_experts is not None else router_w.shape[0]
        self.e_local = w13_q.shape[0]
        self.H, self.I = w2_q.shape[1], w2_q.shape[2]
        self.dev = router_w.device
        self.status = torch.zeros(4, dtype=torch.int32, device=self.dev)
        self._side = None
        # persistent CTAs of the grouped GEMMs (0 = one per SM). A GEMM CTA takes a whole SM (registers and
        # shared memory), so exchanges can only run beside the GEMMs on SMs that are left free.
        self.gemm_ctas = gemm_ctas

    # -- routing and local layout
    def route(self, x):
        T = x.shape[0]
        logits = torch.empty(T, self.E, device=self.dev)
        self.capi.moe_router_logits(logits, x, self.router_w)
        idx = torch.empty(T, self.k, dtype=torch.int32, device=self.dev)
        w = torch.empty(T, self.k, device=self.dev)
        if self.routing == 0:
            self.capi.moe_route_softmax_topk(idx, w, logits)
        else:
            self.capi.moe_route_sigmoid_group_topk(idx, w, logits, self.router_bias, self.n_group, self.topk_group,
                                                   self.scaling)
        return idx, w

    def permute(self, idx):
        tables = self.capi.moe_permute(idx, self.E)
        return tables["counts"], tables["inv_perm"]

    def quant_rows(self, x, inv_perm):
        n = inv_perm.numel()
        rows = torch.empty(n, self.H, dtype=torch.uint8, device=self.dev)
        scales = torch.empty(n, self.H // 128, device=self.dev)
        self.capi.moe_quant_rows(rows, scales, x, inv_perm, self.k)
        return rows, scales

    # -- experts
    def _ffn(self, a_q, a_s, w13_q, w13_s, w2_q, w2_s, tile_expert, num_tiles, max_tiles, status):
        cap, I, H = a_q.shape[0], self.I, self.H
        h_q = torch.empty(cap, I, dtype=torch.uint8, device=self.dev)
        h_s = torch.empty(I // 128, cap, device=self.dev)
        y = torch.empty(cap, H, dtype=torch.bfloat16, device=self.dev)
        self.capi.moe_grouped_gemm_fp8(0, h_q, h_s, a_q, a_s, w13_q, w13_s, tile_expert, num_tiles, max_tiles,
                                       status[0:1], self.gemm_ctas)
        self.capi.moe_grouped_gemm_fp8(1, y, None, h_q, h_s, w2_q, w2_s, tile_expert, num_tiles, max_tiles,
                                       status[1:2], self.gemm_ctas)
        return y

    def expert_ffn(self, recv_rows, recv_scales, plan: ExchangePlan):
        cap, n = plan.rows_cap, recv_rows.shape[0]
        i32 = dict(dtype=torch.int32, device=self.dev)
        a_q = torch.empty(cap, self.H, dtype=torch.uint8, device=self.dev)
        a_s = torch.empty(self.H // 128, cap, device=self.dev)
        self.capi.moe_scatter_rows(a_q, a_s, recv_rows, recv_scales, plan.dst_row)
        max_tiles = cap // 128
        offsets, pad_offsets = torch.empty(self.e_local + 1, **i32), torch.empty(self.e_local + 1, **i32)
        tile_expert, num_tiles = torch.empty(max_tiles, **i32), torch.empty(1, **i32)
        self.capi.moe_tiles_from_counts(plan.local_counts.to(self.dev), offsets, pad_offsets, tile_expert, num_tiles)
        y = self._ffn(a_q, a_s, self.w13_q, self.w13_s, self.w2_q, self.w2_s, tile_expert, num_tiles, max_tiles,
                      self.status[0:2])
        y_recv = torch.empty(n, self.H, dtype=torch.bfloat16, device=self.dev)
        self.capi.moe_gather_rows(y_recv, y, plan.dst_row)
        return y_recv

    # -- merged form: one copy of a token per destination rank
    def quant_copies(self, x, copy_pos, n_copies):
        """copy_pos int32 [T, N]: row of token t's copy for rank d in the send buffer, or -1."""
        rows = torch.empty(n_copies, self.H, dtype=torch.uint8, device=self.dev)
        scales = torch.empty(n_copies, self.H // 128, device=self.dev)
        self.capi.moe_quant_rows(rows, scales, x, copy_pos.reshape(-1), copy_pos.shape[1])
        return rows, scales

    def expert_ffn_entries(self, recv_rows, recv_scales, src_copy, local_counts, cap):
        """src_copy int32 [cap]: received copy behind every row of the padded row space (-1 = padding).
        Returns y bf16 [cap, H] in that row space."""
        i32 = dict(dtype=torch.int32, device=self.dev)
        a_q = torch.empty(cap, self.H, dtype=torch.uint8, device=self.dev)
        # the row gather moves 16-byte pieces: e4m3 rows are handed over as bf16 rows of half the length
        if recv_rows.shape[0]:
            self.capi.moe_gather_rows(a_q.view(torch.bfloat16), recv_rows.view(torch.bfloat16), src_copy)
            a_s = recv_scales[src_copy.clamp(min=0).long()].t().contiguous()
        else:                                     # nothing arrived: one tile of padding
            a_q.zero_()
            a_s = torch.ones(self.H // 128, cap, device=self.dev)
        max_tiles = cap // 128
        offsets, pad_offsets = torch.empty(self.e_local + 1, **i32), torch.empty(self.e_local + 1, **i32)
        tile_expert, num_tiles = torch.empty(max_tiles, **i32), torch.empty(1, **i32)
        self.capi.moe_tiles_from_counts(local_counts.contiguous(), offsets, pad_offsets, tile_expert, num_tiles)
        return self._ffn(a_q, a_s, self.w13_q, self.w13_s, self.w2_q, self.w2_s, tile_expert, num_tiles, max_tiles,
                         self.status[0:2])

    def shared_expert(self, x):
        if self.shared is None:
            return None
        w13_q, w13_s, w2_q, w2_s = self.shared
        T = x.shape[0]
        tiles = (T + 127) // 128
        a_q = torch.empty(tiles * 128, self.H, dtype=torch.uint8, device=self.dev)
        a_s = torch.empty(self.H // 128, tiles * 128, device=self.dev)
        self.capi.moe_quant_dispatch(a_q, a_s, x, None, 1)
        return self._ffn(a_q, a_s, w13_q.unsqueeze(0), w13_s.unsqueeze(0), w2_q.unsqueeze(0), w2_s.unsqueeze(0),
                         None, None, tiles, self.status[2:4])

    def shared_expert_begin(self, x):
        """Shared expert on a side stream; returns what shared_expert_end needs to join it."""
        if self.shared is None:
            return None
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.dev)
        cur = torch.cuda.current_stream(self.dev)
        self._side.wait_stream(cur)
        with torch.cuda.stream(self._side):
            y = self.shared_expert(x)
            x.record_stream(self._side)
        return y

    def shared_expert_end(self, pending):
        if pending is None:
            return None
        cur = torch.cuda.current_stream(self.dev)
        cur.wait_stream(self._side)
        pending.record_stream(cur)
        return pending

    def combine(self, y_back, inv_perm, w, shared):
        T = w.shape[0]
        out = torch.empty(T, self.H, dtype=torch.bfloat16, device=self.dev)
        self.capi.moe_combine(out, y_back, inv_perm, w, shared)
        return out


class PeerLayer:
    """The layer with its exchanges done by the kernels themselves over peer memory (`moe_ep_peer_*` in the
    C ABI): a token's quantised row is stored straight into the receive buffer of every rank that holds one
    of its experts, and the weighted partial results are stored straight back. Capacities are fixed when the
    object is built, so `forward` allocates only its output and never synchronises with the host.

    One process per GPU: the ranks exchange 64-byte CUDA IPC handles of their exchange buffers through
    `group` (a torch.distributed group; any backend that moves bytes). Several ranks of ONE process (tests
    on a single GPU, or one process driving several GPUs) are built with `PeerLayer.build_local`."""

    def __init__(self, ops: CudaOps, rank: int, world: int, t_cap: int, group=None, entry_cap=None, _connect=True):
        import ctypes
        from . import capi
        self.ops, self.rank, self.world, self.t_cap = ops, rank, world, t_cap
        self.capi, self.lib = capi, capi.lib()
        assert ops.E % world == 0 and ops.e_local == ops.E // world
        # entries this rank can receive per call: everything when alone, else 1.5 x the balanced share
        self.entry_cap = entry_cap or (t_cap * ops.k if world == 1 else (t_cap * ops.k * 3) // 2)
        self.ctx = ctypes.c_void_p()
        local_error = None
        try:
            self._create_local(ops, rank, world, t_cap)
        except Exception as exc:  # noqa: BLE001  (reported below, on every rank)
            local_error = exc
        if _connect and world > 1:
            # a rank that could not build its side still answers here, so that the others do not wait for it
            errors = [None] * world
            dist.all_gather_object(errors, None if local_error is None else repr(local_error), group=group)
            bad = {r: e for r, e in enumerate(errors) if e is not None}
            if bad:
                raise RuntimeError(f"expert-parallel layer could not be built on rank(s) {bad}")
        elif local_error is not None:
            raise local_error
        if _connect:
            self._connect_ipc(group)

    def _create_local(self, ops, rank, world, t_cap):
        import ctypes
        capi = self.capi
        with torch.cuda.device(ops.dev):
            capi._check("moe_ep_peer_create",
                        self.lib.moe_ep_peer_create(ctypes.byref(self.ctx), rank, world, t_cap, ops.H, ops.k,
                                                    ops.e_local))
        sh = ops.shared or (None, None, None, None)
        p = lambda t: None if t is None else t.data_ptr()
        self.args = capi.MoeEpLayerArgs(p(ops.router_w), p(ops.router_bias), p(ops.w13_q), p(ops.w13_s), p(ops.w2_q),
                                        p(ops.w2_s), p(sh[0]), p(sh[1]), p(sh[2]), p(sh[3]), ops.E, ops.I, ops.routing,
                                        ops.n_group, ops.topk_group, float(ops.scaling), self.entry_cap, ops.gemm_ctas)
        nbytes = self.lib.moe_ep_peer_workspace_bytes(self.ctx, ctypes.byref(self.args))
        if nbytes == 0:
            raise ValueError("moe_ep_peer_workspace_bytes rejected the layer's shapes")
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=ops.dev)

    def _connect_ipc(self, group):
        """Swap the buffers' IPC handles and map the peers'. A rank whose export or mapping fails still takes
        part in both exchanges and every rank raises, so that no rank is left waiting in a collective."""
        import ctypes
        mine = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.ops.dev):
            rc = self.lib.moe_ep_peer_export(self.ctx, mine)
        if self.world == 1:
            self.capi._check("moe_ep_peer_export", rc)
            handles = bytes(mine)
        else:
            gathered = [None] * self.world
            dist.all_gather_object(gathered, (rc, bytes(mine)), group=group)
            bad = [r for r, (code, _) in enumerate(gathered) if code != 0]
            if bad:
                raise RuntimeError(f"moe_ep_peer_export failed on rank(s) {bad}")
            handles = b"".join(h for _, h in gathered)
        with torch.cuda.device(self.ops.dev):
            rc = self.lib.moe_ep_peer_connect_ipc(self.ctx, handles)
        if self.world > 1:
            codes = [None] * self.world
            dist.all_gather_object(codes, rc, group=group)
            bad = [r for r, code in enumerate(codes) if code != 0]
            if bad:
                raise RuntimeError(f"moe_ep_peer_connect_ipc failed on rank(s) {bad}")
        else:
            self.capi._check("moe_ep_peer_connect_ipc", rc)

    @staticmethod
    def build_local(ops_per_rank, t_cap: int, entry_cap=None):
        """All ranks inside this process (each `ops` on its own device, or all on one)."""
        import ctypes
        world = len(ops_per_rank)
        layers = [PeerLayer(o, r, world, t_cap, entry_cap=entry_cap, _connect=False) for r, o in enumerate(ops_per_rank)]
        table = (ctypes.c_void_p * world)(*[l.ctx.value for l in layers])
        for l in layers:
            with torch.cuda.device(l.ops.dev):
                l.capi._check("moe_ep_peer_connect_local", l.lib.moe_ep_peer_connect_local(l.ctx, table))
        return layers

    def forward(self, x: torch.Tensor, out: torch.Tensor = None, stages: int = 0) -> torch.Tensor:
        """One layer call. `stages` (bit 0: routing + dispatch + shared expert, bit 1: receive + GEMMs + return,
        bit 2: combine; 0 = all) is for ranks that share one GPU, which are stepped stage by stage."""
        import ctypes
        T = x.shape[0]
        if out is None:
            out = torch.empty(T, self.ops.H, dtype=torch.bfloat16, device=x.device)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        with torch.cuda.device(x.device):
            self.capi._check("moe_ep_peer_layer_launcher",
                             self.lib.moe_ep_peer_layer_launcher(self.ctx, out.data_ptr(), x.data_ptr(), T,
                                                                 ctypes.byref(self.args), self.workspace.data_ptr(),
                                                                 self.workspace.numel(), stages, stream))
        return out

    @staticmethod
    def forward_local(layers, xs):
        """One layer call of every rank of `build_local`, stage by stage; returns the outputs in rank order."""
        outs = [torch.empty(x.shape[0], l.ops.H, dtype=torch.bfloat16, device=x.device) for l, x in zip(layers, xs)]
        for stage in (1, 2, 4):
            for l, x, o in zip(layers, xs, outs):
                l.forward(x, o, stage)
        return outs

    def status_codes(self) -> list:
        import ctypes
        host = (ctypes.c_int * 8)()
        with torch.cuda.device(self.ops.dev):
            self.capi._check("moe_ep_peer_read_status",
                             self.lib.moe_ep_peer_read_status(self.ctx, ctypes.byref(self.args),
                                                              self.workspace.data_ptr(), host))
        return list(host)

    def debug_read(self, which: int, numel: int, dtype, offset_bytes: int = 0) -> torch.Tensor:
        out = torch.empty(numel, dtype=dtype, device=self.ops.dev)
        with torch.cuda.device(self.ops.dev):
            self.capi._check("moe_ep_peer_debug_read",
                             self.lib.moe_ep_peer_debug_read(self.ctx, which, offset_bytes, out.data_ptr(),
                                                             out.numel() * out.element_size()))
        return out

    def describe(self) -> str:
        return ("rows stored into the peers' receive buffers by the dispatch kernel and partial results stored back "
                "by the return kernel (peer memory over NVLink, release/acquire flags, no collective call, no host sync)")

    def launches_per_call(self) -> int:
        return 19 + (3 if self.ops.shared is not None else 0)

    def close(self) -> None:
        if self.ctx:
            with torch.cuda.device(self.ops.dev):
                self.lib.moe_ep_peer_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class NcclLayer:
    """The layer with its exchanges made by NCCL all-to-all calls (`ep_moe_forward`): the baseline form."""

    def __init__(self, ops: CudaOps, world: int, group=None, dedup=None, micro_batches: int = 1):
        self.ops, self.world, self.group, self.dedup, self.micro_batches = ops, world, group, dedup, micro_batches

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ep_moe_forward(x, self.ops, self.world, self.group, self.micro_batches, self.dedup)

    def status_codes(self) -> list:
        return self.ops.status.cpu().tolist()

    def describe(self) -> str:
        return "NCCL all-to-all dispatch/return, one copy of a token per destination rank"

    def launches_per_call(self) -> int:
        return 14

    def close(self) -> None:
        pass


def make_layer(ops: CudaOps, rank: int, world: int, t_cap: int, mode: str = "peer", group=None):
    """The expert-parallel layer object for this rank: `.forward(x)` runs one layer call.

    mode "peer": rows are pushed into the other ranks' receive buffers by the kernels themselves
    (`PeerLayer`); mode "nccl": the exchanges are NCCL all-to-all calls (`NcclLayer`)."""
    if mode == "nccl":
        return NcclLayer(ops, world, group)
    if mode == "peer":
        return PeerLayer(ops, rank, world, t_cap, group)
    raise ValueError(f"unknown expert-parallel mode {mode!r}")
