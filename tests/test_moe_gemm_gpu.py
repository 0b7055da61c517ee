"""GPU parity of the tcgen05 grouped FP8 GEMM against the oracle's dequantised fp32 matmul.

Tolerances: the fp32 partial sums only differ by summation order, so the bf16 down
projection must sit within rel-L2 3e-3 (bf16 output rounding) of the oracle; the
re-quantised h may flip single e4m3 codes at rounding boundaries, so it is compared
after dequantisation at rel-L2 1e-2 and its scales at 1e-5 relative.
"""
import pytest
import torch

from conftest import load_oracle

pytestmark = pytest.mark.gpu


def make_rows(m, rows, K, gen, dev):
    x = torch.randn(rows, K, generator=gen)
    q, s = m.quant_1x128(x)
    return q, s, q.view(torch.uint8).to(dev), s.t().contiguous().to(dev)


def check_status(status):
    torch.cuda.synchronize()
    assert int(status) == 0, f"kernel wait gave up at code {int(status)}"


# the last two: the down projection of the expert-parallel layer (N 7168, K 2048) and 56 K blocks (K 7168), where
# the per-lane weight-scale registers use their second half
@pytest.mark.parametrize("rows,N,K", [(128, 256, 128), (128, 256, 512), (256, 512, 1024), (384, 2048, 1024),
                                      (256, 7168, 2048), (128, 512, 7168)])
def test_dense_down_projection(cuda_device, rows, N, K):
    from cuda_agent_b200 import capi
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    gen = torch.Generator().manual_seed(rows + N + K)
    q, s, q_d, st_d = make_rows(m, rows, K, gen, cuda_device)
    wq, ws = m.quant_128x128(torch.randn(1, N, K, generator=gen) * 0.02)
    ref = m.dequant_1x128(q, s) @ m.dequant_128x128(wq[0], ws[0]).t()
    out = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    status = torch.ones(1, dtype=torch.int32, device=cuda_device)
    capi.moe_grouped_gemm_fp8(1, out, None, q_d, st_d, wq.view(torch.uint8).to(cuda_device), ws.to(cuda_device),
                              None, None, rows // 128, status)
    check_status(status)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    rel = float((got - ref).norm() / ref.norm())
    assert rel < 3e-3, rel


# the last one: gate/up of the expert-parallel layer (I 2048, K 7168 = 56 K blocks)
@pytest.mark.parametrize("rows,I,K", [(128, 128, 128), (256, 256, 512), (128, 1024, 2048), (256, 2048, 7168)])
def test_dense_gate_up_swiglu_requant(cuda_device, rows, I, K):
    from cuda_agent_b200 import capi
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    gen = torch.Generator().manual_seed(rows + I + K)
    q, s, q_d, st_d = make_rows(m, rows, K, gen, cuda_device)
    wq, ws = m.quant_128x128(torch.randn(1, 2 * I, K, generator=gen) * 0.05)
    gu = m.dequant_1x128(q, s) @ m.dequant_128x128(wq[0], ws[0]).t()
    h = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    hq_ref, hs_ref = m.quant_1x128(h)
    hq = torch.zeros(rows, I, dtype=torch.uint8, device=cuda_device)
    hs = torch.zeros(I // 128, rows, device=cuda_device)
    status = torch.ones(1, dtype=torch.int32, device=cuda_device)
    capi.moe_grouped_gemm_fp8(0, hq, hs, q_d, st_d, wq.view(torch.uint8).to(cuda_device), ws.to(cuda_device),
                              None, None, rows // 128, status)
    check_status(status)
    hs_cpu = hs.cpu().t().contiguous()
    torch.testing.assert_close(hs_cpu, hs_ref, rtol=1e-4, atol=1e-9)
    got = m.dequant_1x128(hq.cpu().view(torch.float8_e4m3fn), hs_cpu)
    want = m.dequant_1x128(hq_ref, hs_ref)
    assert float((got - want).norm() / want.norm()) < 1e-2
    assert float((hq.cpu() != hq_ref.view(torch.uint8)).float().mean()) < 2e-3   # boundary flips only


@pytest.mark.parametrize("T,H,I,E,k", [(96, 256, 128, 8, 2), (300, 512, 256, 16, 4), (1024, 2048, 1024, 64, 6)])
def test_grouped_pipeline_matches_oracle(cuda_device, T, H, I, E, k):
    """permute -> quantise+dispatch -> GEMM mode 0 -> GEMM mode 1 -> combine, against Model.forward."""
    from cuda_agent_b200 import capi
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    model = m.Model(T, H, I, E, k)
    gen = torch.Generator().manual_seed(T)
    x = torch.randn(T, H, generator=gen).to(torch.bfloat16)
    idx, w = model.route(model.logits(x))
    ref = model(x)
    dev = cuda_device
    perm = capi.moe_permute(idx.to(dev), E)
    cap = perm["max_tiles"] * 128
    a_q = torch.empty(cap, H, dtype=torch.uint8, device=dev)
    a_s = torch.empty(H // 128, cap, device=dev)
    capi.moe_quant_dispatch(a_q, a_s, x.to(dev), perm["dst_row"], k)
    hq = torch.empty(cap, I, dtype=torch.uint8, device=dev)
    hs = torch.empty(I // 128, cap, device=dev)
    y = torch.empty(cap, H, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    capi.moe_grouped_gemm_fp8(0, hq, hs, a_q, a_s, model.w13_q.view(torch.uint8).to(dev), model.w13_s.to(dev),
                              perm["tile_expert"], perm["num_tiles"], perm["max_tiles"], status[0:1])
    capi.moe_grouped_gemm_fp8(1, y, None, hq, hs, model.w2_q.view(torch.uint8).to(dev), model.w2_s.to(dev),
                              perm["tile_expert"], perm["num_tiles"], perm["max_tiles"], status[1:2])
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    capi.moe_combine(out, y, perm["dst_row"], w.to(dev))
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0]
    rel = float((out.float().cpu() - ref.float()).norm() / ref.float().norm())
    assert rel < 2e-2, rel


def test_bounded_wait_gives_up_and_the_kernel_returns(cuda_device):
    """The wait protocol of the tensor-core kernels: an arrival that never comes makes the wait run out after
    its cycle limit; the kernel records the give-up code, goes through its teardown (tensor memory freed) and
    returns, and the device keeps working. With the arrival present the same kernel reports 0."""
    from cuda_agent_b200 import capi
    status = torch.full((1,), -1, dtype=torch.int32, device=cuda_device)
    capi.wait_selftest(status, 200_000, withhold=False)
    torch.cuda.synchronize()
    assert int(status) == 0
    capi.wait_selftest(status, 200_000, withhold=True)       # about 0.1 ms at 1.9 GHz
    torch.cuda.synchronize()
    assert int(status) == 901
    # tensor memory was released and the context is healthy: a real GEMM runs right after
    capi.wait_selftest(status, 200_000, withhold=False)
    torch.cuda.synchronize()
    assert int(status) == 0
    test_dense_down_projection(cuda_device, 128, 256, 128)


def test_one_process_drives_two_gpus(cuda_device):
    """Kernel attributes (the opt-in to large dynamic shared memory) are kept per device: the same process runs
    the tensor-core kernels on device 0 and then on device 1."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on the box")
    from test_mla_gpu import run as run_mla
    m = load_oracle("mla", {"CAB_MLA_CONFIG": 0})
    gen = torch.Generator().manual_seed(3)
    q, kv, seq_len, idx = m.make_inputs(2, 128, 300, 128, 100, gen)
    ref = m.Model(2, 128, 300, 128)(q, kv, seq_len, idx)
    for index in (0, 1):
        dev = torch.device("cuda", index)
        with torch.cuda.device(dev):
            test_dense_down_projection(dev, 128, 256, 512)
            test_dense_gate_up_swiglu_requant(dev, 128, 128, 128)
            for config in (0, 1):
                out = run_mla(dev, q, kv, seq_len, idx, 2, config)
                assert float((out.float() - ref.float()).abs().max()) <= 2e-2
