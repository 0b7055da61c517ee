"""CPU pins for the sparse MLA oracle (oracle/mla/model.py): float64 loops and hand cases."""
import numpy as np
import torch

from conftest import load_oracle


def mla_f64(q, kv, seq_len, idx):
    B, _, Hh, D = q.shape
    out = np.zeros((B, 1, Hh, 512))
    for b in range(B):
        rows = [int(i) for i in idx[b, 0].tolist() if 0 <= int(i) < int(seq_len[b])]
        if not rows:
            continue
        K = kv[b, rows].double().numpy()
        for h in range(Hh):
            s = K @ q[b, 0, h].double().numpy() / np.sqrt(192.0)
            p = np.exp(s - s.max()); p /= p.sum()
            out[b, 0, h] = p @ K[:, :512]
    return out


def test_matches_float64_restatement():
    m = load_oracle("mla", {"CAB_MLA_CONFIG": 0})
    m.reseed()
    q, kv, seq_len, idx = m.get_inputs()
    idx[1, 0, 5:9] = -1                      # padded entries
    idx[2, 0, 0] = int(seq_len[2])           # one past the end -> invalid
    idx[2, 0, 1] = 10 ** 6
    out = m.Model(*m.get_init_inputs())(q, kv, seq_len, idx)
    ref = mla_f64(q, kv, seq_len, idx)
    assert out.shape == (3, 1, 16, 512) and out.dtype == torch.bfloat16
    assert np.abs(out.double().numpy() - ref).max() < 2e-2
    assert np.abs(out.double().numpy() - ref).max() < 0.01 * np.abs(ref).max() + 4e-3   # bf16 rounding only


def test_matches_float64_restatement_at_the_benchmark_shape():
    """Two sequences of the benchmark's shape (128 heads, 2048 of up to 32768 cached rows) against the float64 loop."""
    m = load_oracle("mla", {"CAB_MLA_CONFIG": 2})
    q, kv, seq_len, idx = m.make_inputs(2, 128, 32768, 2048, 8192, torch.Generator().manual_seed(31))
    idx[1, 0, 100:140] = -1
    out = m.Model(*m.get_init_inputs())(q, kv, seq_len, idx)
    ref = mla_f64(q, kv, seq_len, idx)
    assert out.shape == (2, 1, 128, 512)
    assert np.abs(out.double().numpy() - ref).max() < 0.01 * np.abs(ref).max() + 4e-3   # bf16 rounding only


def test_hand_cases():
    m = load_oracle("mla", {"CAB_MLA_CONFIG": 0})
    kv = torch.zeros(1, 8, 576, dtype=torch.bfloat16)
    kv[0, 2, :512] = 1.0
    kv[0, 5, :512] = 3.0
    q = torch.zeros(1, 1, 2, 576, dtype=torch.bfloat16)
    model = m.Model(1, 2, 8, 4)
    # zero query: uniform weights over the two valid rows -> (1 + 3) / 2
    idx = torch.tensor([[[2, 5, -1, 9]]], dtype=torch.int32)
    out = model(q, kv, torch.tensor([8], dtype=torch.int32), idx)
    assert torch.all(out == 2.0)
    # a single valid row is returned as is, whatever its score
    out = model(q, kv, torch.tensor([4], dtype=torch.int32), idx)
    assert torch.all(out == 1.0)
    # no valid row -> zeros
    out = model(q, kv, torch.tensor([2], dtype=torch.int32), idx)
    assert torch.all(out == 0.0)
    # gather: invalid entries are zero rows, valid ones are the cache rows bit for bit
    rows = m.gather_rows(kv, idx, torch.tensor([8], dtype=torch.int32))
    assert torch.equal(rows[0, 0], kv[0, 2]) and torch.equal(rows[0, 1], kv[0, 5])
    assert torch.all(rows[0, 2] == 0) and torch.all(rows[0, 3] == 0)


def test_inputs_follow_the_stated_distributions():
    m = load_oracle("mla", {"CAB_MLA_CONFIG": 0})
    m.reseed()
    q, kv, seq_len, idx = m.get_inputs()
    assert q.shape == (3, 1, 16, 576) and kv.shape == (3, 300, 576) and idx.shape == (3, 1, 64)
    for b in range(3):
        chosen = idx[b, 0][idx[b, 0] >= 0]
        assert len(set(chosen.tolist())) == len(chosen)                 # sampled without replacement
        assert int(chosen.max()) < int(seq_len[b])
        assert len(chosen) == min(64, int(seq_len[b]))


def test_several_query_tokens_per_sequence():
    """Sq > 1: every token is the one-token operator on the shared cache with its own selection and length."""
    m = load_oracle("mla", {"CAB_MLA_CONFIG": 0})
    gen = torch.Generator().manual_seed(77)
    B, Sq, Hh, S, topk = 2, 3, 4, 90, 32
    _, kv, _, _ = m.make_inputs(B, Hh, S, topk, 40, gen)
    q = torch.randn(B, Sq, Hh, 576, generator=gen).to(torch.bfloat16)
    seq_len = torch.tensor([[50, 51, 52], [88, 89, 90]], dtype=torch.int32)
    idx = torch.randint(-2, S + 3, (B, Sq, topk), generator=gen, dtype=torch.int32)
    out = m.Model(B, Hh, S, topk)(q, kv, seq_len, idx)
    assert out.shape == (B, Sq, Hh, 512)
    for s in range(Sq):
        ref = mla_f64(q[:, s:s + 1], kv, seq_len[:, s], idx[:, s:s + 1])
        assert np.abs(out[:, s:s + 1].double().numpy() - ref).max() < 0.01 * np.abs(ref).max() + 4e-3
    # a [B] seq_len applies to every token of the sequence
    out1 = m.Model(B, Hh, S, topk)(q, kv, seq_len[:, 0].contiguous(), idx)
    ref = mla_f64(q[:, 2:3], kv, seq_len[:, 0], idx[:, 2:3])
    assert np.abs(out1[:, 2:3].double().numpy() - ref).max() < 0.01 * np.abs(ref).max() + 4e-3


def test_matches_committed_fixture():
    """tests/golden/mla_small.npz (written by tests/golden/make_mla_moe_golden.py) pins the oracle over time."""
    import importlib.util
    from conftest import GOLDEN
    spec = importlib.util.spec_from_file_location("make_mla_moe_golden", GOLDEN / "make_mla_moe_golden.py")
    gen_mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen_mod)
    fix = np.load(GOLDEN / "mla_small.npz")
    m = load_oracle("mla", {"CAB_MLA_CONFIG": 0})
    for heads in (64, 128):
        q, kv, seq_len, idx = gen_mod.mla_case(m, heads)
        out = m.Model(2, heads, 300, 128)(q, kv, seq_len, idx)
        got = out.reshape(-1)[::int(fix["stride"])].float().numpy()
        want = torch.from_numpy(fix[f"out{heads}"].view(np.int16)).view(torch.bfloat16).float().numpy()
        # the same arithmetic; a different thread count may move a sum by one bf16 step
        assert np.mean(got == want) > 0.99
        assert np.abs(got - want).max() <= 2.0 ** -7 * np.abs(want).max()

