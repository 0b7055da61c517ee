"""CPU pins for the GDN oracle (oracle/gdn/model.py).

The reference has no GDN vector, so the oracle is pinned here by (1) an
independent float64 restatement that forms the dk x dk matrix (I - beta k k^T)
explicitly, (2) hand-computable cases, (3) the committed fixture.
"""
import numpy as np
import pytest
import torch

from conftest import GOLDEN, load_oracle


def gdn_step_f64(S, q, k, v, g, beta, group):
    """Literal S' = alpha S (I - beta k k^T) + beta v k^T; o = S' q / sqrt(dk), float64 loops."""
    B, Hv, dv, dk = S.shape
    S_new = np.empty_like(S, dtype=np.float64)
    o = np.empty((B, Hv, dv), dtype=np.float64)
    eye = np.eye(dk)
    for b in range(B):
        for h in range(Hv):
            kk = k[b, h // group].astype(np.float64)
            qq = q[b, h // group].astype(np.float64)
            vv = v[b, h].astype(np.float64)
            alpha = np.exp(np.float64(g[b, h]))
            bt = np.float64(beta[b, h])
            M = eye - bt * np.outer(kk, kk)
            S_new[b, h] = alpha * (S[b, h].astype(np.float64) @ M) + bt * np.outer(vv, kk)
            o[b, h] = S_new[b, h] @ qq / np.sqrt(dk)
    return o, S_new


def to_np(t):
    return t.float().numpy()


@pytest.mark.parametrize("B,Hq,Hv", [(1, 1, 1), (2, 2, 4), (3, 4, 4)])
def test_oracle_matches_float64_restatement(B, Hq, Hv):
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 0})
    gen = torch.Generator().manual_seed(7 + B)
    S = m.make_state(B, Hv, gen)
    q, k, v, g, beta = m.make_step_inputs(B, Hq, Hv, gen)
    o, S_new = m.Model(B, Hq, Hv)(S, q, k, v, g, beta)
    o64, S64 = gdn_step_f64(to_np(S), to_np(q), to_np(k), to_np(v), to_np(g), to_np(beta), Hv // Hq)
    assert np.linalg.norm(o.numpy() - o64) / np.linalg.norm(o64) < 2e-6
    assert np.linalg.norm(S_new.numpy() - S64) / np.linalg.norm(S64) < 2e-6


def test_oracle_hand_case_one_hot_key():
    """k = e_3, q = e_3: column 3 of S becomes alpha*(1-beta)*S[:,3] + beta*v, others scale by alpha."""
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 0})
    D = m.D
    S = torch.arange(D * D, dtype=torch.float32).reshape(1, 1, D, D) / (D * D)
    k = torch.zeros(1, 1, D); k[0, 0, 3] = 1.0
    q = k.clone()
    v = torch.linspace(-1, 1, D).reshape(1, 1, D).to(torch.bfloat16)
    g = torch.tensor([[-0.5]]); beta = torch.tensor([[0.25]])
    o, S_new = m.Model(1, 1, 1)(S, q.bfloat16(), k.bfloat16(), v, g, beta)
    alpha = float(np.exp(-0.5))
    expect = alpha * S.clone()
    expect[0, 0, :, 3] = alpha * (1 - 0.25) * S[0, 0, :, 3] + 0.25 * v.float()[0, 0]
    torch.testing.assert_close(S_new, expect, rtol=1e-6, atol=1e-7)
    torch.testing.assert_close(o[0, 0], expect[0, 0, :, 3] / D ** 0.5, rtol=1e-6, atol=1e-7)


def test_oracle_identities():
    """beta = 0 -> pure decay; g = 0, beta = 1, S = 0 -> S' = v k^T and o = v (k.q)/sqrt(d)."""
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 0})
    gen = torch.Generator().manual_seed(3)
    S = m.make_state(2, 2, gen)
    q, k, v, g, _ = m.make_step_inputs(2, 2, 2, gen)
    zero = torch.zeros(2, 2)
    o, S_new = m.Model(2, 2, 2)(S, q, k, v, g, zero)
    torch.testing.assert_close(S_new, torch.exp(g)[..., None, None] * S, rtol=1e-6, atol=1e-9)
    o2, S2 = m.Model(2, 2, 2)(torch.zeros_like(S), q, k, v, zero, torch.ones(2, 2))
    torch.testing.assert_close(S2, v.float()[..., :, None] * k.float()[..., None, :], rtol=1e-6, atol=1e-9)
    kq = (k.float() * q.float()).sum(-1, keepdim=True)
    torch.testing.assert_close(o2, v.float() * kq / m.D ** 0.5, rtol=1e-5, atol=1e-8)


def test_inputs_follow_the_stated_distributions():
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 0})
    m.reseed()
    S, q, k, v, g, beta = m.get_inputs()
    assert S.shape == (4, 8, 128, 128) and S.dtype == torch.float32
    assert q.shape == k.shape == (4, 8, 128) and q.dtype == k.dtype == torch.bfloat16
    assert v.shape == (4, 8, 128) and v.dtype == torch.bfloat16
    assert g.shape == beta.shape == (4, 8) and g.dtype == torch.float32
    assert abs(float(S.std()) - 0.02) < 1e-3
    torch.testing.assert_close(q.float().norm(dim=-1), torch.ones(4, 8), atol=1e-2, rtol=0)
    assert (g < 0).all() and ((beta > 0) & (beta < 1)).all()
    m.reseed()
    again = m.get_inputs()
    assert all(torch.equal(a, b) for a, b in zip([S, q, k, v, g, beta], again))


def test_oracle_reproduces_committed_fixture():
    fix = np.load(GOLDEN / "gdn_config0.npz")
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 0})
    m.reseed(int(fix["seed"]))
    o, S_new = m.Model(*m.get_init_inputs())(*m.get_inputs())
    np.testing.assert_allclose(o.numpy(), fix["o"], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(S_new.flatten()[:: int(fix["stride"])].numpy(), fix["state_sample"],
                               rtol=1e-5, atol=1e-8)


def test_config1_shapes():
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 1})
    assert m.get_init_inputs() == [256, 16, 32]
