"""CPU pins for the MoE oracle (oracle/moe/model.py).

The reference has no MoE vector, so the oracle is pinned by: e4m3 known-answer
values against a table-driven rounding written here from the format definition;
an independent float64 per-token restatement of the whole layer; hand-made
routing and permutation cases.
"""
import numpy as np
import pytest
import torch

from conftest import load_oracle


# --------------------------------------------------------------------------- e4m3 from its definition
def e4m3_table():
    """All finite e4m3 (fn variant: bias 7, no inf, 0x7F/0xFF are NaN) values by code."""
    vals = np.full(256, np.nan)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        exp, man = (code >> 3) & 0xF, code & 0x7
        if exp == 0xF and man == 0x7:
            continue
        vals[code] = sign * (man / 8.0 * 2.0 ** -6 if exp == 0 else (1 + man / 8.0) * 2.0 ** (exp - 7))
    return vals


def e4m3_round_rne(v: np.ndarray) -> np.ndarray:
    """Nearest representable value, ties to the even mantissa code, saturating at 448."""
    table = e4m3_table()
    pos = np.sort(table[:127][~np.isnan(table[:127])])      # 0 .. 448, ascending == code order
    a = np.minimum(np.abs(v.astype(np.float64)), 448.0)
    hi = np.searchsorted(pos, a, side="left").clip(0, len(pos) - 1)
    lo = (hi - 1).clip(0)
    d_lo, d_hi = a - pos[lo], pos[hi] - a
    pick = np.where(d_lo < d_hi, lo, np.where(d_hi < d_lo, hi, np.where(lo % 2 == 0, lo, hi)))
    return np.sign(v) * pos[pick]


def test_e4m3_known_answers():
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    table = e4m3_table()
    assert table[0x7E] == 448.0 and table[0x01] == 2.0 ** -9 and table[0x08] == 2.0 ** -6
    # representable, half-way (ties to even), saturating and tiny values
    probes = np.array([0.0, 1.0, 1.0625, 1.125, 1.1875, 17.0, 18.0, 19.0, 20.0, 21.0, 22.0, 447.9, 448.0,
                       460.0, 1e4, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10, 1e-4, -0.3, -300.0, -449.0],
                      dtype=np.float32)
    got = torch.from_numpy(probes).clamp(-448, 448).to(torch.float8_e4m3fn).float().numpy()
    np.testing.assert_array_equal(got, e4m3_round_rne(probes).astype(np.float32))
    # 1x128 rule end to end on random data
    gen = torch.Generator().manual_seed(0)
    v = torch.randn(5, 256, generator=gen) * 3
    q, s = m.quant_1x128(v)
    blocks = v.numpy().reshape(5, 2, 128)
    amax = np.maximum(np.abs(blocks).max(-1), 1e-4).astype(np.float32)
    scale = (amax / np.float32(448.0)).astype(np.float32)
    np.testing.assert_array_equal(s.numpy(), scale)
    expect = e4m3_round_rne((blocks / scale[..., None]).astype(np.float32))
    np.testing.assert_array_equal(q.float().numpy().reshape(5, 2, 128), expect.astype(np.float32))
    assert float(q.float().abs().max()) == 448.0


def test_weight_quant_is_per_128x128_block():
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    gen = torch.Generator().manual_seed(1)
    w = torch.randn(2, 256, 384, generator=gen) * 0.02
    q, s = m.quant_128x128(w)
    assert q.shape == w.shape and s.shape == (2, 2, 3)
    blk = w[1, 128:256, 256:384]
    assert float(s[1, 1, 2]) == float(blk.abs().max() / 448.0)
    back = m.dequant_128x128(q, s)
    assert float((back - w).norm() / w.norm()) < 0.04


# --------------------------------------------------------------------------- routing
def test_softmax_routing_hand_cases():
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    logits = torch.tensor([[0.0, 2.0, 1.0, 2.0, -1.0, 0.5, 2.0, 0.0],
                           [1.0] * 8])
    idx, w = m.route_softmax_topk(logits, 3)
    assert idx.tolist() == [[1, 3, 6], [0, 1, 2]]          # ties -> lower expert id
    torch.testing.assert_close(w, torch.full((2, 3), 1 / 3))
    idx, w = m.route_softmax_topk(torch.tensor([[0.0, 1.0, 3.0, 2.0]]), 2)
    assert idx.tolist() == [[2, 3]]
    e = np.exp([0.0, -1.0]); torch.testing.assert_close(w[0], torch.tensor(e / e.sum(), dtype=torch.float32))
    # equivalent to ordering by the full softmax
    gen = torch.Generator().manual_seed(2)
    big = torch.randn(50, 64, generator=gen)
    idx, w = m.route_softmax_topk(big, 6)
    p = torch.softmax(big.double(), -1)
    ref = torch.sort(p, dim=-1, descending=True, stable=True)
    assert torch.equal(idx.long(), ref.indices[:, :6])
    torch.testing.assert_close(w.double(), ref.values[:, :6] / ref.values[:, :6].sum(-1, keepdim=True),
                               rtol=1e-5, atol=1e-7)


def test_sigmoid_group_routing_hand_case():
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 1})
    # 8 experts, 4 groups of 2, keep 2 groups, top-3
    logits = torch.tensor([[3.0, -3.0, 2.0, 2.0, 0.0, 0.0, 2.5, -1.0]])
    bias = torch.zeros(8)
    s = torch.sigmoid(logits.double()).float()[0]
    # group scores: g0 = s0+s1, g1 = 2*s(2.0), g2 = 1.0, g3 = s(2.5)+s(-1)
    scores = [float(s[0] + s[1]), float(s[2] + s[3]), float(s[4] + s[5]), float(s[6] + s[7])]
    keep = sorted(np.argsort([-x for x in scores], kind="stable")[:2].tolist())
    assert keep == [1, 3]
    idx, w = m.route_sigmoid_group_topk(logits, bias, 3, 4, 2, routed_scaling_factor=2.0)
    assert idx.tolist() == [[6, 2, 3]]
    chosen = s[[6, 2, 3]]
    torch.testing.assert_close(w[0], chosen / chosen.sum() * 2.0)
    # the bias moves selection but not the weights
    bias2 = torch.tensor([0.0, 0.0, 0.0, 0.0, 5.0, 5.0, 0.0, 0.0])
    idx2, w2 = m.route_sigmoid_group_topk(logits, bias2, 2, 4, 1)
    assert idx2.tolist() == [[4, 5]]
    torch.testing.assert_close(w2[0], torch.tensor([0.5, 0.5]))


def test_permutation_is_a_stable_sort():
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    idx = torch.tensor([[2, 0], [1, 2], [0, 2], [2, 1]], dtype=torch.int32)
    perm, inv, counts = m.permutation(idx, 4)
    assert perm.tolist() == [1, 4, 2, 7, 0, 3, 5, 6]
    assert counts.tolist() == [2, 2, 4, 0]
    assert [inv[p] for p in perm.tolist()] == list(range(8))


# --------------------------------------------------------------------------- whole layer vs float64
def layer_f64(model, x):
    """Token-by-token float64 restatement with the table-driven e4m3 rounding above."""
    m_T, H = x.shape
    I, k = model.I, model.k
    idx, w = model.route(model.logits(x))
    deq = lambda q, s: np.kron(s.double().numpy(), np.ones((128, 128))) * q.double().numpy()

    def quant_rows(v):
        blocks = v.reshape(v.shape[0], -1, 128)
        amax = np.maximum(np.abs(blocks).max(-1), 1e-4).astype(np.float32)
        scale = (amax / np.float32(448.0)).astype(np.float32)
        q = e4m3_round_rne((blocks.astype(np.float32) / scale[..., None]).astype(np.float32))
        return (q * scale[..., None].astype(np.float64)).reshape(v.shape)

    def ffn(a, w13, w2):
        gu = a @ w13.T
        g, u = gu[:, :I], gu[:, I:]
        h = g / (1 + np.exp(-g)) * u
        y = quant_rows(h) @ w2.T
        return torch.from_numpy(y).to(torch.bfloat16).double().numpy()

    a = quant_rows(x.float().numpy())
    out = np.zeros((m_T, H))
    W13 = [deq(model.w13_q[e], model.w13_s[e]) for e in range(model.E)]
    W2 = [deq(model.w2_q[e], model.w2_s[e]) for e in range(model.E)]
    for t in range(m_T):
        for slot in range(k):
            e = int(idx[t, slot])
            out[t] += float(w[t, slot]) * ffn(a[t:t + 1], W13[e], W2[e])[0]
    if model.has_shared:
        out += ffn(a, deq(model.shared_w13_q, model.shared_w13_s), deq(model.shared_w2_q, model.shared_w2_s))
    return out


@pytest.mark.parametrize("cfg", [0, 1])
def test_layer_matches_float64_restatement(cfg):
    m = load_oracle("moe", {"CAB_MOE_CONFIG": cfg})
    m.reseed()
    model = m.Model(*m.get_init_inputs())
    (x,) = m.get_inputs()
    x = x[:24]
    out = model(x).double().numpy()
    ref = layer_f64(model, x)
    rel = np.linalg.norm(out - ref) / np.linalg.norm(ref)
    assert rel < 6e-3, rel        # bf16 output rounding (~2e-3) + rare e4m3 boundary flips of h
    assert np.isfinite(out).all() and np.abs(out).max() > 0


def test_layer_matches_float64_restatement_at_benchmark_width():
    """The same check with the benchmark layer's H 2048 / I 1024 (16 and 8 scale blocks per row) and top-6 of
    8 experts: the float64 restatement is independent of the oracle's blocked fp32 arithmetic."""
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 0})
    torch.manual_seed(99)
    model = m.Model(12, 2048, 1024, 8, 6, "softmax", 1, 1, False)
    x = torch.randn(12, 2048, generator=torch.Generator().manual_seed(98)).to(torch.bfloat16)
    out = model(x).double().numpy()
    ref = layer_f64(model, x)
    rel = np.linalg.norm(out - ref) / np.linalg.norm(ref)
    assert rel < 6e-3, rel
    assert np.isfinite(out).all() and np.abs(out).max() > 0


def test_state_dict_names():
    m = load_oracle("moe", {"CAB_MOE_CONFIG": 1})
    model = m.Model(*m.get_init_inputs())
    names = set(model.state_dict())
    assert {"router_w", "router_bias", "w13_q", "w13_s", "w2_q", "w2_s", "shared_w13_q", "shared_w13_s",
            "shared_w2_q", "shared_w2_s"} == names
    assert model.w13_q.dtype == torch.float8_e4m3fn and model.w13_s.shape == (16, 4, 2)


@pytest.mark.parametrize("cfg", [0, 1])
def test_matches_committed_fixture(cfg):
    """tests/golden/moe_config{cfg}.npz (written by tests/golden/make_mla_moe_golden.py) pins the oracle over time."""
    from conftest import GOLDEN
    fix = np.load(GOLDEN / f"moe_config{cfg}.npz")
    m = load_oracle("moe", {"CAB_MOE_CONFIG": cfg})
    m.reseed()
    (x,) = m.get_inputs()
    model = m.Model(*m.get_init_inputs())
    idx, w = model.route(model.logits(x))
    assert np.array_equal(idx.numpy().astype(np.int32), fix["idx"])
    np.testing.assert_allclose(w.numpy(), fix["w"], rtol=1e-5, atol=1e-7)
    out = model(x).float().numpy()
    want = torch.from_numpy(fix["out"].view(np.int16)).view(torch.bfloat16).float().numpy()
    assert np.linalg.norm(out - want) <= 1e-3 * np.linalg.norm(want)

