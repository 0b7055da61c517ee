"""GPU parity of the MoE routing / permutation / quantise-dispatch / combine kernels.

Integer and byte outputs (expert indices, permutation tables, e4m3 bytes, fp32
scales) must be identical to the oracle's; fp32 routing weights within 1e-5
relative; logits and the bf16 combine within fp32 summation-order noise.
"""
import pytest
import torch

from conftest import load_oracle

pytestmark = pytest.mark.gpu


def i32(*shape, dev):
    return torch.full(shape, -7, dtype=torch.int32, device=dev)


# batches of 512 tokens and more with E % 32 == 0 take the tcgen05 kernel (config 0), the rest and config 1 mma.sync
@pytest.mark.parametrize("T,H,E", [(96, 256, 8), (33, 512, 64), (4096, 2048, 64), (70, 7168, 256), (16, 64, 72),
                                   (1100, 7168, 256), (513, 128, 32), (640, 2048, 96)])
def test_router_logits(cuda_device, T, H, E):
    from cuda_agent_b200 import capi
    gen = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, H, generator=gen).to(torch.bfloat16)
    wr = (torch.randn(E, H, generator=gen) * 0.02).to(torch.bfloat16)
    ref = x.double() @ wr.double().t()
    for config in (0, 1):
        out = torch.full((T, E), float("nan"), device=cuda_device)
        capi.moe_router_logits(out, x.to(cuda_device), wr.to(cuda_device), config)
        err = (out.cpu().double() - ref).abs().max()
        assert float(err) < 2e-5 * float(ref.abs().max()) + 1e-6, (config, float(err))


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (96, 8, 2), (4096, 64, 6), (1000, 256, 8), (50, 40, 5), (17, 64, 32)])
def test_softmax_topk_exact(cuda_device, T, E, k):
    from cuda_agent_b200 import capi
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    gen = torch.Generator().manual_seed(E * 1000 + k)
    logits = torch.randn(T, E, generator=gen)
    logits[::3] = logits[::3].round()                      # many exact ties
    if T > 2:
        logits[2] = 1.0                                    # all equal
    ref_idx, ref_w = m.route_softmax_topk(logits, k)
    idx, w = i32(T, k, dev=cuda_device), torch.empty(T, k, device=cuda_device)
    capi.moe_route_softmax_topk(idx, w, logits.to(cuda_device))
    assert torch.equal(idx.cpu(), ref_idx)
    torch.testing.assert_close(w.cpu(), ref_w, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("T,E,k,ng,tg", [(80, 16, 4, 4, 2), (8192, 256, 8, 8, 4), (64, 8, 3, 4, 2), (33, 64, 6, 1, 1),
                                         (40, 256, 8, 32, 5)])
def test_sigmoid_group_topk_exact(cuda_device, T, E, k, ng, tg):
    from cuda_agent_b200 import capi
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 1})
    gen = torch.Generator().manual_seed(E + k)
    logits = torch.randn(T, E, generator=gen)
    logits[::4] = (logits[::4] * 2).round() / 2            # ties in s and in group scores
    bias = torch.randn(E, generator=gen) * 0.02
    bias[::2] = 0.0
    ref_idx, ref_w = m.route_sigmoid_group_topk(logits, bias, k, ng, tg, 2.5)
    idx, w = i32(T, k, dev=cuda_device), torch.empty(T, k, device=cuda_device)
    capi.moe_route_sigmoid_group_topk(idx, w, logits.to(cuda_device), bias.to(cuda_device), ng, tg, 2.5)
    assert torch.equal(idx.cpu(), ref_idx), int((idx.cpu() != ref_idx).sum())
    torch.testing.assert_close(w.cpu(), ref_w, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("T,k,E", [(4, 2, 4), (96, 2, 8), (4096, 6, 64), (8192, 8, 256), (1, 1, 1), (1025, 3, 5),
                                   (300, 4, 256)])
def test_permutation_exact(cuda_device, T, k, E):
    from cuda_agent_b200 import capi
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    gen = torch.Generator().manual_seed(T * 7 + E)
    # k distinct experts per token, skewed so that some experts stay empty
    scores = torch.rand(T, E, generator=gen) + (torch.arange(E) % 3 == 0) * 0.5
    idx = scores.topk(min(k, E), dim=-1).indices.to(torch.int32)
    if idx.shape[1] < k:
        idx = idx.repeat(1, k)[:, :k].contiguous()
    perm, inv, counts = m.permutation(idx, E)
    for _ in range(2):                                      # second call reuses nothing stale
        res = capi.moe_permute(idx.to(cuda_device), E)
        torch.cuda.synchronize()
        assert torch.equal(res["counts"].cpu(), counts)
        assert torch.equal(res["perm"].cpu(), perm) and torch.equal(res["inv_perm"].cpu(), inv)
        offsets = torch.cat([torch.zeros(1, dtype=torch.int64), counts.long().cumsum(0)])
        assert torch.equal(res["offsets"].cpu().long(), offsets)
        tiles = (counts.long() + 127) // 128
        pad = torch.cat([torch.zeros(1, dtype=torch.int64), (tiles * 128).cumsum(0)])
        assert torch.equal(res["pad_offsets"].cpu().long(), pad)
        flat = idx.reshape(-1).long()
        expect_dst = pad[flat] + (inv.long() - offsets[flat])
        assert torch.equal(res["dst_row"].cpu().long(), expect_dst)
        nt = int(tiles.sum())
        assert int(res["num_tiles"]) == nt
        assert torch.equal(res["tile_expert"].cpu()[:nt].long(), torch.repeat_interleave(torch.arange(E), tiles))
        assert bool((res["tile_expert"].cpu()[nt:] == -1).all())
        assert int(res["scratch"].view(torch.int32)[-1]) == 0


def test_permutation_flags_bad_expert_ids(cuda_device):
    from cuda_agent_b200 import capi
    idx = torch.tensor([[0, 9], [1, 2]], dtype=torch.int32, device=cuda_device)
    res = capi.moe_permute(idx, 4)
    torch.cuda.synchronize()
    assert int(res["scratch"].view(torch.int32)[-1]) == 1
    assert res["counts"].cpu().tolist() == [1, 1, 1, 0]


def test_permutation_skips_invalid_entries(cuda_device):
    """Entries without a valid expert (-1 from a router that ran out of finite candidates, ids >= E) get
    no row: inv_perm = dst_row = -1, the tail of perm is -1, the rest is the stable sort of the valid ones."""
    from cuda_agent_b200 import capi
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    gen = torch.Generator().manual_seed(3)
    T, k, E = 700, 4, 16
    idx = torch.randint(0, E, (T, k), generator=gen, dtype=torch.int32)
    idx[5] = -1                                  # a token with no expert at all
    idx[::7, 2] = -1
    idx[300, 0] = E + 3
    valid = (idx >= 0) & (idx < E)
    flat_valid = valid.reshape(-1)
    # oracle on the valid entries only, mapped back to flat positions
    keys = idx.reshape(-1)[flat_valid]
    order = torch.argsort(keys.long(), stable=True)
    where = torch.nonzero(flat_valid).reshape(-1)
    perm_ref = torch.full((T * k,), -1, dtype=torch.int32); perm_ref[: len(order)] = where[order].to(torch.int32)
    inv_ref = torch.full((T * k,), -1, dtype=torch.int32); inv_ref[where[order]] = torch.arange(len(order), dtype=torch.int32)
    counts = torch.bincount(keys.long(), minlength=E)
    for config, flag in ((0, 1), (1, 1)):        # the id E + 3 is flagged either way
        res = capi.moe_permute(idx.to(cuda_device), E, config)
        torch.cuda.synchronize()
        assert torch.equal(res["counts"].cpu().long(), counts)
        assert torch.equal(res["perm"].cpu(), perm_ref) and torch.equal(res["inv_perm"].cpu(), inv_ref)
        dst = res["dst_row"].cpu()
        assert bool((dst[~flat_valid] == -1).all()) and bool((dst[flat_valid] >= 0).all())
        assert int(res["scratch"].view(torch.int32)[-1]) == flag
    idx[300, 0] = 1                              # only -1 markers left: flagged without config bit 0, silent with it
    assert int(capi.moe_permute(idx.to(cuda_device), E, 0)["scratch"].view(torch.int32)[-1]) == 1
    assert int(capi.moe_permute(idx.to(cuda_device), E, 1)["scratch"].view(torch.int32)[-1]) == 0


def test_nan_token_is_dropped_without_stray_writes(cuda_device):
    """A NaN activation row leaves the router without candidates (-1 in every slot). Its entries must get
    no row: nothing is written outside the padded row space and the token's combined output is zero."""
    from cuda_agent_b200 import capi
    gen = torch.Generator().manual_seed(8)
    T, H, E, k = 40, 256, 8, 2
    x = torch.randn(T, H, generator=gen).to(torch.bfloat16)
    x[7] = float("nan")
    wr = (torch.randn(E, H, generator=gen) * 0.02).to(torch.bfloat16)
    dev = cuda_device
    logits = torch.empty(T, E, device=dev)
    capi.moe_router_logits(logits, x.to(dev), wr.to(dev))
    idx, w = i32(T, k, dev=dev), torch.empty(T, k, device=dev)
    capi.moe_route_softmax_topk(idx, w, logits)
    assert idx[7].cpu().tolist() == [-1] * k
    res = capi.moe_permute(idx, E)
    assert int(res["scratch"].view(torch.int32)[-1]) == 1
    assert res["dst_row"].view(T, k)[7].cpu().tolist() == [-1] * k
    cap, guard = res["max_tiles"] * 128, 8
    big_q = torch.full((cap + 2 * guard, H), 0xAA, dtype=torch.uint8, device=dev)
    big_s = torch.full((H // 128, cap + 2 * guard), -1.0, device=dev)
    # the row space is a view with poisoned guard rows on both sides
    capi.moe_quant_dispatch(big_q[guard:], big_s, x.to(dev), res["dst_row"], k)
    torch.cuda.synchronize()
    assert bool((big_q[:guard] == 0xAA).all()) and bool((big_q[guard + cap:] == 0xAA).all())
    written = (big_q[guard:guard + cap] != 0xAA).any(dim=1).sum()
    assert int(written) <= (T - 1) * k
    y = torch.randn(cap, H, generator=gen).to(torch.bfloat16).to(dev)
    out = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device=dev)
    capi.moe_combine(out, y, res["dst_row"], torch.nan_to_num(w), None)
    assert bool((out[7] == 0).all()) and bool(torch.isfinite(out.float()).all())


def test_permutation_of_an_empty_batch(cuda_device):
    """T = 0 with 256 experts: the tables are written for zero entries and nothing past the scratch
    size the library asks for is touched."""
    from cuda_agent_b200 import capi
    E, k = 256, 8
    lib = capi.lib()
    need = lib.moe_permute_scratch_bytes(0, k, E)
    assert need >= (E + 2) * 4
    guard = 4096
    buf = torch.full((need + guard,), 0x5C, dtype=torch.uint8, device=cuda_device)
    i32k = dict(dtype=torch.int32, device=cuda_device)
    counts, offsets, pad = torch.full((E,), -7, **i32k), torch.full((E + 1,), -7, **i32k), torch.full((E + 1,), -7, **i32k)
    max_tiles = lib.moe_permute_max_tiles(0, k, E)
    tile_expert, num_tiles = torch.full((max_tiles,), -7, **i32k), torch.full((1,), -7, **i32k)
    rc = lib.moe_permute_launcher(None, 0, k, E, counts.data_ptr(), offsets.data_ptr(), pad.data_ptr(), None, None,
                                  None, tile_expert.data_ptr(), num_tiles.data_ptr(), max_tiles, buf.data_ptr(), 0,
                                  torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0
    assert bool((buf[need:] == 0x5C).all())
    assert int(counts.abs().sum()) == 0 and int(offsets.abs().sum()) == 0 and int(pad.abs().sum()) == 0
    assert int(num_tiles) == 0 and bool((tile_expert == -1).all())


@pytest.mark.parametrize("T,H,k", [(96, 256, 2), (40, 2048, 6), (9, 7168, 8), (5, 128, 1), (33, 384, 3)])
def test_quant_dispatch_exact(cuda_device, T, H, k):
    from cuda_agent_b200 import capi
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    gen = torch.Generator().manual_seed(H + k)
    x = (torch.randn(T, H, generator=gen) * torch.logspace(-3, 1, T)[:, None]).to(torch.bfloat16)
    x[0, :128] = 0                                          # an all-zero block hits the amax floor
    q_ref, s_ref = m.quant_1x128(x.float())
    # plain quantisation (dst_row = NULL)
    a_q = torch.zeros(T, H, dtype=torch.uint8, device=cuda_device)
    sc = torch.zeros(H // 128, T, device=cuda_device)
    capi.moe_quant_dispatch(a_q, sc, x.to(cuda_device), None, 1)
    assert torch.equal(a_q.cpu(), q_ref.view(torch.uint8))
    assert torch.equal(sc.cpu().t().contiguous(), s_ref)
    # dispatch to k scattered rows each
    rows = T * k + 64
    dst = torch.randperm(rows, generator=gen)[: T * k].to(torch.int32).reshape(T, k)
    a_q = torch.full((rows, H), 0xAA, dtype=torch.uint8, device=cuda_device)
    sc = torch.full((H // 128, rows), -1.0, device=cuda_device)
    capi.moe_quant_dispatch(a_q, sc, x.to(cuda_device), dst.to(cuda_device), k)
    a_cpu, sc_cpu = a_q.cpu(), sc.cpu()
    for slot in range(k):
        assert torch.equal(a_cpu[dst[:, slot].long()], q_ref.view(torch.uint8))
        assert torch.equal(sc_cpu[:, dst[:, slot].long()].t().contiguous(), s_ref)
    untouched = torch.ones(rows, dtype=torch.bool); untouched[dst.reshape(-1).long()] = False
    assert bool((a_cpu[untouched] == 0xAA).all()) and bool((sc_cpu[:, untouched] == -1.0).all())


@pytest.mark.parametrize("T,H,k,extra", [(96, 256, 2, False), (64, 2048, 6, False), (10, 7168, 8, True), (3, 8, 1, True)])
def test_combine(cuda_device, T, H, k, extra):
    from cuda_agent_b200 import capi
    gen = torch.Generator().manual_seed(T + H)
    rows = T * k + 17
    y = torch.randn(rows, H, generator=gen).to(torch.bfloat16)
    dst = torch.randperm(rows, generator=gen)[: T * k].to(torch.int32).reshape(T, k)
    w = torch.rand(T, k, generator=gen)
    ex = torch.randn(T, H, generator=gen).to(torch.bfloat16) if extra else None
    ref = torch.zeros(T, H)
    for slot in range(k):
        ref = ref + w[:, slot, None] * y[dst[:, slot].long()].float()
    if extra:
        ref = ref + ex.float()
    out = torch.empty(T, H, dtype=torch.bfloat16, device=cuda_device)
    capi.moe_combine(out, y.to(cuda_device), dst.to(cuda_device), w.to(cuda_device),
                     ex.to(cuda_device) if extra else None)
    # fma vs mul+add differs below bf16 resolution except at rounding boundaries
    torch.testing.assert_close(out.cpu().float(), ref.to(torch.bfloat16).float(), rtol=8e-3, atol=1e-3)
    assert float((out.cpu().float() - ref).norm() / ref.norm()) < 3e-3
