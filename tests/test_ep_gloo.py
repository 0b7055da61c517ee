"""Expert-parallel bookkeeping on CPU: ExchangePlan by hand, and the full EP schedule over gloo with
world_size 2, the compute steps replaced by the oracle's functions, against the single-process oracle."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, load_oracle


def test_exchange_plan_hand_case():
    from cuda_agent_b200.ep import ExchangePlan
    # 2 ranks, 2 local experts each. I send [[3,0],[1,2]]; I receive [[3,0],[130,1]] for my experts (0,1).
    send = torch.tensor([[3, 0], [1, 2]])
    recv = torch.tensor([[3, 0], [130, 1]])
    plan = ExchangePlan.from_matrices(send, recv)
    assert plan.send_splits == [3, 3] and plan.recv_splits == [3, 131]
    assert plan.local_counts.tolist() == [133, 1]
    assert plan.rows_cap == 256 + 128                      # expert 0 needs two tiles, expert 1 one
    dst = plan.dst_row.tolist()
    assert dst[:3] == [0, 1, 2]                            # source 0, expert 0
    assert dst[3:133] == list(range(3, 133))               # source 1, expert 0 follows source 0's rows
    assert dst[133] == 256                                 # source 1, expert 1 starts at the padded offset
    assert len(set(dst)) == len(dst) == 134


class OracleOps:
    """The ops contract of cuda_agent_b200.ep on CPU, built from the oracle's functions."""

    def __init__(self, m, model, rank, world):
        self.m, self.model, self.rank, self.world = m, model, rank, world
        self.e_local = model.E // world

    def route(self, x):
        return self.model.route(self.model.logits(x))

    def permute(self, idx):
        perm, inv, counts = self.m.permutation(idx, self.model.E)
        return counts, inv

    def quant_rows(self, x, inv_perm):
        q, s = self.m.quant_1x128(x.float())
        k = self.model.k
        rows = torch.empty(inv_perm.numel(), x.shape[1], dtype=torch.uint8)
        scales = torch.empty(inv_perm.numel(), x.shape[1] // 128)
        token = torch.arange(inv_perm.numel()) // k
        rows[inv_perm.long()] = q.view(torch.uint8)[token]
        scales[inv_perm.long()] = s[token]
        return rows, scales

    def expert_ffn(self, recv_rows, recv_scales, plan):
        padded = (plan.local_counts.long() + 127) // 128 * 128
        ends = torch.cumsum(padded, 0)
        expert = torch.searchsorted(ends, plan.dst_row.long(), right=True)
        y = torch.empty(recv_rows.shape[0], self.model.H, dtype=torch.bfloat16)
        for e in range(self.e_local):
            sel = (expert == e).nonzero().flatten()
            if sel.numel():
                ge = self.rank * self.e_local + e
                y[sel] = self.m.expert_ffn(recv_rows[sel].view(torch.float8_e4m3fn), recv_scales[sel],
                                           self.model.w13_q[ge], self.model.w13_s[ge], self.model.w2_q[ge],
                                           self.model.w2_s[ge]).to(torch.bfloat16)
        return y

    def quant_copies(self, x, copy_pos, n_copies):
        q, s = self.m.quant_1x128(x.float())
        rows = torch.empty(n_copies, x.shape[1], dtype=torch.uint8)
        scales = torch.empty(n_copies, x.shape[1] // 128)
        t, d = (copy_pos >= 0).nonzero(as_tuple=True)
        rows[copy_pos[t, d].long()] = q.view(torch.uint8)[t]
        scales[copy_pos[t, d].long()] = s[t]
        return rows, scales

    def expert_ffn_entries(self, recv_rows, recv_scales, src_copy, local_counts, cap):
        padded = (local_counts.long() + 127) // 128 * 128
        starts = torch.cumsum(padded, 0) - padded
        y = torch.zeros(cap, self.model.H, dtype=torch.bfloat16)
        for e in range(self.e_local):
            n = int(local_counts[e])
            if n:
                sel = src_copy[int(starts[e]):int(starts[e]) + n].long()
                ge = self.rank * self.e_local + e
                y[int(starts[e]):int(starts[e]) + n] = self.m.expert_ffn(
                    recv_rows[sel].view(torch.float8_e4m3fn), recv_scales[sel], self.model.w13_q[ge],
                    self.model.w13_s[ge], self.model.w2_q[ge], self.model.w2_s[ge]).to(torch.bfloat16)
        return y

    def shared_expert(self, x):
        if not self.model.has_shared:
            return None
        q, s = self.m.quant_1x128(x.float())
        return self.m.expert_ffn(q, s, self.model.shared_w13_q, self.model.shared_w13_s, self.model.shared_w2_q,
                                 self.model.shared_w2_s).to(torch.bfloat16)

    def combine(self, y_back, inv_perm, w, shared):
        T, k = w.shape
        rows = inv_perm.long().reshape(T, k)
        ys = y_back[rows.clamp(min=0)].float()                     # [T, k, H]; negative rows are empty slots
        out = torch.zeros(T, ys.shape[-1])
        for slot in range(k):
            out = out + torch.where(rows[:, slot, None] >= 0, w[:, slot, None] * ys[:, slot], torch.zeros(()))
        if shared is not None:
            out = out + shared.float()
        return out.to(torch.bfloat16)


def _worker(rank, world, port, cfg, result_dir):
    # cfg 1 also exercises the two-micro-batch schedule (every rank must issue the same collectives)

    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cuda_agent_b200.ep import ep_moe_forward
        torch.set_num_threads(2)
        m = load_oracle("moe", {"CAB_MOE_CONFIG": cfg})
        model = m.Model(*m.get_init_inputs())
        gen = torch.Generator().manual_seed(100 + rank)
        T = 70 + 13 * rank                                  # ragged: ranks hold different token counts
        x = torch.randn(T, model.H, generator=gen).to(torch.bfloat16)
        ops = OracleOps(m, model, rank, world)
        out = ep_moe_forward(x, ops, world, micro_batches=1 + cfg, dedup=False)     # one row per (token, slot)
        merged = ep_moe_forward(x, ops, world)                                      # one row per (token, rank)
        ref = model(x)
        rel = float((out.float() - ref.float()).norm() / ref.float().norm())
        rel_merged = float((merged.float() - ref.float()).norm() / ref.float().norm())
        torch.save({"rel": rel, "rel_merged": rel_merged, "T": T}, os.path.join(result_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cfg", [0, 1])
def test_ep_schedule_over_gloo_world2(tmp_path, cfg):
    port = 29600 + cfg + (os.getpid() % 200)
    mp.spawn(_worker, args=(2, port, cfg, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        res = torch.load(tmp_path / f"rank{rank}.pt")
        assert res["rel"] < 2e-3, res                      # same arithmetic, only bf16 rounding order differs
        assert res["rel_merged"] < 6e-3, res               # + one bf16 rounding of the partial sum per (token, rank)


def test_ep_schedule_over_gloo_world4(tmp_path):
    """Four ranks, 16 experts in 4 groups (one group per rank), top-4 over 2 groups: a token reaches at most two
    ranks, so the merged form sends at most two copies where the per-entry form sends four rows."""
    port = 29850 + (os.getpid() % 100)
    mp.spawn(_worker, args=(4, port, 1, str(tmp_path)), nprocs=4, join=True)
    for rank in range(4):
        res = torch.load(tmp_path / f"rank{rank}.pt")
        assert res["rel"] < 2e-3, res
        assert res["rel_merged"] < 6e-3, res

