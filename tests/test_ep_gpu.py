"""Expert-parallel MoE on GPUs: the world_size-1 path on one GPU (same kernels, no exchange) and, when the
box has two GPUs, two NCCL ranks, each against the eager oracle on its own tokens (rel-L2 2e-2)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, load_oracle

pytestmark = pytest.mark.gpu


def make_ops(model, dev, rank, world):
    from cuda_agent_b200.ep import CudaOps
    el = model.E // world
    sl = slice(rank * el, (rank + 1) * el)
    g = lambda t: t.to(dev).contiguous()
    shared = None
    if model.has_shared:
        shared = (g(model.shared_w13_q), g(model.shared_w13_s), g(model.shared_w2_q), g(model.shared_w2_s))
    return CudaOps(g(model.router_w.data), g(model.router_bias), g(model.w13_q[sl]), g(model.w13_s[sl]),
                   g(model.w2_q[sl]), g(model.w2_s[sl]), shared, k=model.k,
                   routing=0 if model.routing == "softmax" else 1, n_group=model.n_group,
                   topk_group=model.topk_group, scaling=model.routed_scaling_factor, num_experts=model.E)


@pytest.mark.parametrize("cfg,T", [(0, 96), (1, 80), (1, 300)])
def test_world1_matches_oracle_and_fused_op(cuda_device, cfg, T):
    import cuda_agent_b200
    from cuda_agent_b200.ep import ep_moe_forward
    m = load_oracle("moe", {"CAB_MOE_CONFIG": cfg})
    args = m.get_init_inputs(); args[0] = T
    model = m.Model(*args)
    ops = make_ops(model, cuda_device, 0, 1)
    x = torch.randn(T, model.H, generator=torch.Generator().manual_seed(T)).to(torch.bfloat16)
    out = ep_moe_forward(x.to(cuda_device), ops, 1, dedup=False)      # one row per (token, expert)
    torch.cuda.synchronize()
    assert ops.status.cpu().tolist()[:2] == [0, 0]
    ref = model(x)
    rel = float((out.float().cpu() - ref.float()).norm() / ref.float().norm())
    assert rel <= 2e-2, rel
    ext = cuda_agent_b200.load_extension()
    sd = {k: v.to(cuda_device) for k, v in model.state_dict().items()}
    sh = [sd.get(n) for n in ("shared_w13_q", "shared_w13_s", "shared_w2_q", "shared_w2_s")]
    fused = ext.moe_forward(x.to(cuda_device), sd["router_w"], sd["router_bias"], sd["w13_q"], sd["w13_s"], sd["w2_q"],
                            sd["w2_s"], *sh, model.k, 0 if model.routing == "softmax" else 1, model.n_group,
                            model.topk_group, 1.0, True, 0)
    assert torch.equal(out, fused)                         # same kernels, same row order per expert
    merged = ep_moe_forward(x.to(cuda_device), ops, 1)                  # default: one copy per (token, rank)
    torch.cuda.synchronize()
    assert ops.status.cpu().tolist()[:2] == [0, 0]
    rel_m = float((merged.float().cpu() - ref.float()).norm() / ref.float().norm())
    assert rel_m <= 2e-2, rel_m
    out2 = ep_moe_forward(x.to(cuda_device), ops, 1, micro_batches=2)   # two halves on two streams
    torch.cuda.synchronize()
    assert torch.equal(out2, out)


def _rank_main(rank, world, port, cfg, result_dir):
    sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from cuda_agent_b200.ep import ep_moe_forward
        m = load_oracle("moe", {"CAB_MOE_CONFIG": cfg})
        model = m.Model(*m.get_init_inputs())
        ops = make_ops(model, dev, rank, world)
        T = 200 + 56 * rank
        x = torch.randn(T, model.H, generator=torch.Generator().manual_seed(7 + rank)).to(torch.bfloat16)
        out = ep_moe_forward(x.to(dev), ops, world, micro_batches=1 + cfg)
        torch.cuda.synchronize()
        ref = model(x)
        rel = float((out.float().cpu() - ref.float()).norm() / ref.float().norm())
        torch.save({"rel": rel, "status": ops.status.cpu().tolist()}, os.path.join(result_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cfg", [0, 1])
def test_two_nccl_ranks(cuda_device, tmp_path, cfg):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on the box")
    port = 29800 + cfg + (os.getpid() % 150)
    mp.spawn(_rank_main, args=(2, port, cfg, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        res = torch.load(tmp_path / f"rank{rank}.pt")
        assert res["status"] == [0, 0, 0, 0] and res["rel"] <= 2e-2, res
