"""Expert-parallel MoE with the exchange done by the kernels over peer memory (PeerLayer).

With fewer GPUs than ranks the ranks live on ONE GPU and are stepped stage by stage (every rank's dispatch is
launched before any rank waits for it), which runs the same kernels, buffers, flags and C orchestration as one
process per GPU does. When the box has two GPUs, two processes exchange CUDA IPC handles and run the layer for
real. Parity: rel-L2 2e-2 against the eager oracle on each rank's own tokens; what a rank receives (rows, scales,
sort keys) is compared bit for bit with the oracle's quantisation and routing.
"""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, load_oracle
from test_ep_gpu import make_ops

pytestmark = pytest.mark.gpu


def rel_l2(got, want):
    return float((got.float().cpu() - want.float()).norm() / want.float().norm())


@pytest.mark.parametrize("cfg,world", [(0, 1), (0, 2), (1, 2), (1, 4), (0, 8), (1, 8)])
def test_virtual_ranks_on_one_gpu(cuda_device, cfg, world):
    from cuda_agent_b200.ep import PeerLayer
    m = load_oracle("moe", {"CAB_MOE_CONFIG": cfg})
    model = m.Model(*m.get_init_inputs())
    dev = cuda_device
    ops = [make_ops(model, dev, r, world) for r in range(world)]
    t_cap = 300
    layers = PeerLayer.build_local(ops, t_cap)
    try:
        for call in range(3):                   # later calls reuse every buffer and flag of the earlier ones
            gen = torch.Generator().manual_seed(100 * call + world)
            T_r = [t_cap - 37 * r - 11 * call for r in range(world)]
            if call == 2:
                T_r[-1] = 0                     # a rank without tokens still takes part in both exchanges
            xs = [torch.randn(T, model.H, generator=gen).to(torch.bfloat16) for T in T_r]
            outs = PeerLayer.forward_local(layers, [x.to(dev) for x in xs])
            torch.cuda.synchronize()
            for r in range(world):
                assert layers[r].status_codes() == [0] * 8, (call, r, layers[r].status_codes())
                if T_r[r]:
                    assert rel_l2(outs[r], model(xs[r])) <= 2e-2, (call, r)
        # what rank d holds from source s after the last call: bit-exact against the oracle's routing and quantisation
        el, k, nb = model.E // world, model.k, model.H // 128
        side_ld = nb + 2 * k
        for d in range(world):
            counts = layers[d].debug_read(4, world, torch.int32).cpu().tolist()
            rows = layers[d].debug_read(0, world * t_cap * model.H, torch.uint8).view(world, t_cap, model.H).cpu()
            side = layers[d].debug_read(1, world * t_cap * side_ld, torch.int32).view(world, t_cap, side_ld).cpu()
            for s in range(world):
                if xs[s].shape[0] == 0:
                    assert counts[s] == 0
                    continue
                idx, w = model.route(model.logits(xs[s]))
                here = (idx // el) == d                                   # [T, k]
                tokens = torch.nonzero(here.any(dim=1)).reshape(-1)
                assert counts[s] == len(tokens)
                q, sc = m.quant_1x128(xs[s][tokens].float())
                assert torch.equal(rows[s, : len(tokens)], q.view(torch.uint8))
                assert torch.equal(side[s, : len(tokens), :nb].view(torch.float32), sc)
                want_e = torch.where(here[tokens], idx[tokens] - d * el, torch.full_like(idx[tokens], -1))
                assert torch.equal(side[s, : len(tokens), nb + k:], want_e)
                want_w = torch.where(here[tokens], w[tokens], torch.zeros_like(w[tokens]))
                torch.testing.assert_close(side[s, : len(tokens), nb:nb + k].view(torch.float32), want_w, rtol=1e-5,
                                           atol=1e-7)
    finally:
        for l in layers:
            l.close()


def test_more_entries_than_capacity_are_dropped_and_flagged(cuda_device):
    """entry_cap bounds the rows a rank accepts per call: the overflow is reported (status word 4 = 2), nothing
    is written outside the row space, and the next call with a fitting load is correct again."""
    from cuda_agent_b200.ep import PeerLayer
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    model = m.Model(*m.get_init_inputs())
    ops = [make_ops(model, cuda_device, r, 2) for r in range(2)]
    layers = PeerLayer.build_local(ops, 256, entry_cap=128)
    try:
        gen = torch.Generator().manual_seed(5)
        xs = [torch.randn(256, model.H, generator=gen).to(torch.bfloat16) for _ in range(2)]   # ~512 entries per rank
        outs = PeerLayer.forward_local(layers, [x.to(cuda_device) for x in xs])
        torch.cuda.synchronize()
        assert all(bool(torch.isfinite(o.float()).all()) for o in outs)
        assert any(l.status_codes()[4] == 2 for l in layers)
        xs = [torch.randn(20, model.H, generator=gen).to(torch.bfloat16) for _ in range(2)]    # ~40 entries per rank
        outs = PeerLayer.forward_local(layers, [x.to(cuda_device) for x in xs])
        torch.cuda.synchronize()
        for r in range(2):
            assert layers[r].status_codes() == [0] * 8
            assert rel_l2(outs[r], model(xs[r])) <= 2e-2
    finally:
        for l in layers:
            l.close()


def test_eight_ranks_at_full_dimensions_on_one_gpu(cuda_device):
    """The expert-parallel layer as eight GPUs run it (H 7168, I 2048, 256 experts in blocks of 32, top-8 with
    8 groups / top-4, shared expert), with the eight ranks stepped on one GPU and 256 tokens each: every rank's
    first 48 tokens against the eager oracle."""
    sys.path.insert(0, str(ROOT))
    from bench_workloads import MoeEpWorkload
    from cuda_agent_b200.ep import PeerLayer
    world, T = 8, 256
    wls = [MoeEpWorkload(cuda_device, r, world, T=T, connect=False) for r in range(world)]
    layers = PeerLayer.build_local([w.ops for w in wls], T)
    try:
        for call in range(2):
            outs = PeerLayer.forward_local(layers, [w.x for w in wls])
            torch.cuda.synchronize()
        for r in range(world):
            assert layers[r].status_codes() == [0] * 8, (r, layers[r].status_codes())
            p = wls[r].parity(outs[r], 48)
            assert p["tokens_routed_differently"] <= 1 and p["rel_l2_identically_routed"] <= 2e-2, (r, p)
        # one group of 32 experts per rank: a token travels to topk_group = 4 ranks at most
        counts = torch.stack([l.debug_read(4, world, torch.int32).cpu() for l in layers])     # [dest, source]
        assert world * T * 2 <= int(counts.sum()) <= world * T * 4
    finally:
        for l in layers:
            l.close()


def _rank_main(rank, world, port, cfg, result_dir):
    sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)      # carries the 64-byte handles only
    try:
        from cuda_agent_b200.ep import make_layer
        m = load_oracle("moe", {"CAB_MOE_CONFIG": cfg})
        model = m.Model(*m.get_init_inputs())
        ops = make_ops(model, dev, rank, world)
        layer = make_layer(ops, rank, world, 320, mode="peer")
        rels = []
        for call in range(3):
            T = 200 + 56 * rank + 9 * call
            x = torch.randn(T, model.H, generator=torch.Generator().manual_seed(7 + rank + 10 * call)).to(torch.bfloat16)
            out = layer.forward(x.to(dev))
            torch.cuda.synchronize()
            rels.append(rel_l2(out, model(x)))
        torch.save({"rel": max(rels), "status": layer.status_codes()}, os.path.join(result_dir, f"rank{rank}.pt"))
        dist.barrier()
        layer.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cfg", [0, 1])
def test_two_processes_over_cuda_ipc(cuda_device, tmp_path, cfg):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on the box")
    port = 29950 + cfg + (os.getpid() % 40)
    mp.spawn(_rank_main, args=(2, port, cfg, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        res = torch.load(tmp_path / f"rank{rank}.pt")
        assert res["status"] == [0] * 8 and res["rel"] <= 2e-2, res


def test_task_workspace_passes_the_verification_loop(cuda_device, built_libs, capsys):
    """tasks/moe_ep/model_new.py (one rank: the exchange goes through this GPU's own buffers) against the eager
    model, through the reference-style gate."""
    os.environ["CAB_MOE_CONFIG"] = "1"
    sys.path.insert(0, str(built_libs.WORKDIR))
    from utils import verification
    rc = verification.main(["--task", str(built_libs.WORKDIR / "tasks" / "moe_ep"),
                            "--model-dir", str(ROOT / "oracle" / "moe")])
    assert rc == 0
    assert "[PASS] verify success" in capsys.readouterr().out
