"""GPU parity of the GDN decode kernel against the eager oracle, through the C ABI.

Tolerance (stated for this path): rel 1e-3 on both o and the fp32 state,
checked as rel-L2 <= 1e-3 and |diff| <= 1e-3*(max|ref| + |ref|) elementwise.
"""
import numpy as np
import pytest
import torch

from conftest import GOLDEN, ROOT, load_oracle

pytestmark = pytest.mark.gpu
TOL = 1e-3


def assert_rel(actual, expected, tol=TOL, what=""):
    a, e = actual.double().cpu(), expected.double().cpu()
    assert torch.isfinite(a).all(), what
    rel = float((a - e).norm() / e.norm())
    assert rel <= tol, f"{what}: rel-L2 {rel:.3e}"
    bound = tol * float(e.abs().max()) + tol * e.abs()
    assert bool(((a - e).abs() <= bound).all()), f"{what}: elementwise bound exceeded"


def run_capi(dev, S, q, k, v, g, beta, config=0):
    from cuda_agent_b200 import capi
    Sd = S.to(dev).clone()
    out = torch.full((S.shape[0], S.shape[1], 128), float("nan"), device=dev)
    capi.gdn_decode(Sd, out, q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev), config)
    torch.cuda.synchronize()
    return out, Sd


@pytest.mark.parametrize("config", [0, 1, 2, 3, 4, 16, 19, 17])   # 16: the units walked from last to first
@pytest.mark.parametrize("B,Hq,Hv", [(4, 8, 8), (1, 1, 1), (3, 2, 4), (5, 1, 6), (2, 16, 32)])
def test_matches_oracle(cuda_device, B, Hq, Hv, config):
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 0})
    gen = torch.Generator().manual_seed(100 + 7 * B + Hv)
    S = m.make_state(B, Hv, gen)
    q, k, v, g, beta = m.make_step_inputs(B, Hq, Hv, gen)
    o_ref, S_ref = m.Model(B, Hq, Hv)(S, q, k, v, g, beta)
    o, S_new = run_capi(cuda_device, S, q, k, v, g, beta, config)
    assert_rel(o, o_ref, what="o")
    assert_rel(S_new, S_ref, what="state")


def test_config0_against_committed_fixture(cuda_device):
    fix = np.load(GOLDEN / "gdn_config0.npz")
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 0})
    m.reseed(int(fix["seed"]))
    o, S_new = run_capi(cuda_device, *m.get_inputs())
    assert_rel(o, torch.from_numpy(fix["o"]), what="o vs fixture")
    assert_rel(S_new.flatten()[:: int(fix["stride"])], torch.from_numpy(fix["state_sample"]),
               what="state sample vs fixture")


def test_launch_variants_agree(cuda_device):
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 0})
    gen = torch.Generator().manual_seed(5)
    S = m.make_state(3, 4, gen)
    step = m.make_step_inputs(3, 2, 4, gen)
    results = [run_capi(cuda_device, S, *step, config=c) for c in (4, 1, 2)]      # 128-bit variants
    for o, S_new in results[1:]:
        assert torch.equal(o, results[0][0]) and torch.equal(S_new, results[0][1])
    wide = [run_capi(cuda_device, S, *step, config=c) for c in (0, 3)]            # 256-bit variants
    assert torch.equal(wide[0][0], wide[1][0]) and torch.equal(wide[0][1], wide[1][1])
    torch.testing.assert_close(wide[0][1], results[0][1], rtol=1e-5, atol=1e-7)
    # the direction of the walk changes nothing in the result
    for c in (16, 19):
        o, S_new = run_capi(cuda_device, S, *step, config=c)
        assert torch.equal(o, wide[0][0]) and torch.equal(S_new, wide[0][1]), c
    # an unaligned state falls back to the 128-bit kernel
    from cuda_agent_b200 import capi
    pad = torch.zeros(S.numel() + 4, device=cuda_device)
    view = pad[4:].view_as(S)                      # 16-byte but not 32-byte aligned
    view.copy_(S)
    out = torch.empty(3, 4, 128, device=cuda_device)
    capi.gdn_decode(view, out, *[t.to(cuda_device) for t in step], 0)
    assert torch.equal(view, results[0][1]) and torch.equal(out, results[0][0])


def test_multi_step_recurrence_stays_within_tolerance(cuda_device):
    """16 chained steps: the in-place state must track the oracle's, not drift."""
    from cuda_agent_b200 import capi
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 0})
    B, Hq, Hv = 2, 2, 4
    gen = torch.Generator().manual_seed(11)
    S_ref = m.make_state(B, Hv, gen)
    Sd = S_ref.to(cuda_device).clone()
    out = torch.empty(B, Hv, 128, device=cuda_device)
    model = m.Model(B, Hq, Hv)
    for _ in range(16):
        step = m.make_step_inputs(B, Hq, Hv, gen)
        o_ref, S_ref = model(S_ref, *step)
        capi.gdn_decode(Sd, out, *[t.to(cuda_device) for t in step])
        assert_rel(out, o_ref, what="o")
    assert_rel(Sd, S_ref, what="state after 16 steps")


def test_full_size_zigzag_loop_equals_forward_loop(cuda_device):
    """Eight chained full-size steps (512 MiB of state) with the direction of the walk alternating, against the
    same eight steps walked forwards: bit-identical state and outputs."""
    from cuda_agent_b200 import capi
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 1})
    B, Hq, Hv = m.get_init_inputs()
    dev = cuda_device
    gd = torch.Generator(device=dev).manual_seed(77)
    S0 = torch.randn(B, Hv, 128, 128, device=dev, generator=gd) * 0.02
    gen = torch.Generator().manual_seed(78)
    steps = [[t.to(dev) for t in m.make_step_inputs(B, Hq, Hv, gen)] for _ in range(8)]
    outs = []
    for zigzag in (False, True):
        S = S0.clone()
        o = torch.empty(8, B, Hv, 128, device=dev)
        for i, step in enumerate(steps):
            capi.gdn_decode(S, o[i], *step, capi.gdn_loop_config(i) if zigzag else 0)
        torch.cuda.synchronize()
        outs.append((S, o))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert [capi.gdn_loop_config(i, 3) for i in range(3)] == [3, 19, 3]


def test_full_size_properties(cuda_device):
    """Config 1 (B=256, Hq=16, Hv=32; 512 MiB of state) through size-independent properties.

    * beta = 0: the step is a pure decay, S' = exp(g) S exactly up to fp32 rounding,
      and o = exp(g) S q / sqrt(128) (checked on sampled heads against float64).
    * linearity in the state: step(S1 + S2) - step(S2) = alpha * S1 (I - beta k k^T) has no v term,
      checked on sampled heads.
    * a sampled set of (b, hv) heads equals the oracle run on just those heads.
    """
    from cuda_agent_b200 import capi
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 1})
    B, Hq, Hv = m.get_init_inputs()
    dev = cuda_device
    gen = torch.Generator().manual_seed(1235)
    gd = torch.Generator(device=dev).manual_seed(1235)
    S0 = torch.randn(B, Hv, 128, 128, device=dev, generator=gd) * 0.02
    q, k, v, g, beta = [t.to(dev) for t in m.make_step_inputs(B, Hq, Hv, gen)]
    out = torch.empty(B, Hv, 128, device=dev)

    # (1) pure decay
    S = S0.clone()
    capi.gdn_decode(S, out, q, k, v, g, torch.zeros_like(beta))
    expect = torch.exp(g)[..., None, None] * S0
    assert float((S - expect).norm() / expect.norm()) < 5e-6
    del expect

    # (2) sampled heads against the oracle
    S = S0.clone()
    capi.gdn_decode(S, out, q, k, v, g, beta)
    torch.cuda.synchronize()
    pick_b = torch.tensor([0, 17, 128, 255])
    model = m.Model(len(pick_b), Hq, Hv)
    o_ref, S_ref = model(S0[pick_b].cpu(), q[pick_b].cpu(), k[pick_b].cpu(), v[pick_b].cpu(),
                         g[pick_b].cpu(), beta[pick_b].cpu())
    assert_rel(out[pick_b], o_ref, what="o (sampled batch rows)")
    assert_rel(S[pick_b], S_ref, what="state (sampled batch rows)")

    # (3) every state element was written exactly once per launch: a second identical launch on
    # a fresh copy gives the same bits, and no element kept its input value where alpha != 1.
    S2 = S0.clone()
    out2 = torch.empty_like(out)
    capi.gdn_decode(S2, out2, q, k, v, g, beta)
    assert torch.equal(S2, S) and torch.equal(out2, out)
    assert int((S == S0).sum()) < S.numel() // 10000


def test_full_size_after_1_and_64_steps(cuda_device):
    """Config 1 (B=256, 16/32 heads): 64 chained decode steps with fresh inputs per step; sampled batch
    rows are compared with the oracle stepping just those rows, after step 1 and after step 64."""
    from cuda_agent_b200 import capi
    m = load_oracle("gdn", {"CAB_GDN_CONFIG": 1})
    B, Hq, Hv = m.get_init_inputs()
    dev = cuda_device
    gd = torch.Generator(device=dev).manual_seed(4321)
    S = torch.randn(B, Hv, 128, 128, device=dev, generator=gd) * 0.02
    pick = torch.tensor([0, 101, 255])
    S_ref = S[pick].cpu()
    model = m.Model(len(pick), Hq, Hv)
    out = torch.empty(B, Hv, 128, device=dev)
    gen = torch.Generator().manual_seed(4322)
    for step in range(64):
        inputs = m.make_step_inputs(B, Hq, Hv, gen)
        capi.gdn_decode(S, out, *[t.to(dev) for t in inputs])
        o_ref, S_ref = model(S_ref, *[t[pick] for t in inputs])
        if step in (0, 63):
            assert_rel(out[pick], o_ref, what=f"o after step {step + 1}")
            assert_rel(S[pick], S_ref, what=f"state after step {step + 1}")


def test_extension_and_verification_loop(cuda_device, built_libs, capsys):
    """The reference-style gate: oracle model.py vs tasks/gdn/model_new.py, 5 trials."""
    import sys
    sys.path.insert(0, str(built_libs.WORKDIR))
    from utils import verification
    rc = verification.main(["--task", str(built_libs.WORKDIR / "tasks" / "gdn"),
                            "--model-dir", str(ROOT / "oracle" / "gdn")])
    assert rc == 0
    text = capsys.readouterr().out
    assert "[PASS] check 5/5" in text and "[PASS] verify success" in text


def test_binding_rejects_bad_inputs(cuda_device):
    import cuda_agent_b200
    ext = cuda_agent_b200.load_extension()
    dev = cuda_device
    S = torch.zeros(1, 2, 128, 128, device=dev)
    q = torch.zeros(1, 2, 128, device=dev, dtype=torch.bfloat16)
    v = torch.zeros(1, 2, 128, device=dev, dtype=torch.bfloat16)
    g = torch.zeros(1, 2, device=dev)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ext.gdn_decode_forward(S.cpu(), q, q, v, g, g)
    with pytest.raises(RuntimeError, match="BFloat16"):
        ext.gdn_decode_forward(S, q.float(), q, v, g, g)
    with pytest.raises(RuntimeError, match="multiple of Hq"):
        ext.gdn_decode_forward(S, torch.zeros(1, 3, 128, device=dev, dtype=torch.bfloat16),
                               torch.zeros(1, 3, 128, device=dev, dtype=torch.bfloat16), v, g, g)
    with pytest.raises(RuntimeError, match="contiguous"):
        ext.gdn_decode_forward(S.transpose(2, 3), q, q, v, g, g)


def test_axpby_smoke_op(cuda_device):
    from cuda_agent_b200 import capi
    import cuda_agent_b200
    ext = cuda_agent_b200.load_extension()
    for n in (1, 128, 1000, 4099):
        a = torch.randn(n, device=cuda_device); b = torch.randn(n, device=cuda_device)
        for cfg in (0, 1, 2):
            torch.testing.assert_close(ext.axpby_forward(a, b, 2.0, cfg), 2.0 * a + b, rtol=1e-6, atol=1e-6)
        out = torch.empty_like(a)
        capi.axpby(out[1:], a[1:], b[1:], -0.5)  # misaligned views take the scalar path
        torch.testing.assert_close(out[1:], -0.5 * a[1:] + b[1:], rtol=1e-6, atol=1e-6)


def test_decode_loop_as_cuda_graph(cuda_device, built_libs):
    """Eight steps recorded as one CUDA graph leave the same state and outputs as eight separate launches."""
    from cuda_agent_b200 import capi
    from cuda_agent_b200.graphs import GdnDecodeGraph
    gen = torch.Generator().manual_seed(5)
    B, Hq, Hv, steps = 4, 8, 8, 8
    state0 = (torch.randn(B, Hv, 128, 128, generator=gen) * 0.02).to(cuda_device)
    def unit(x):
        return (x / x.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
    q = unit(torch.randn(steps, B, Hq, 128, generator=gen)).to(cuda_device)
    k = unit(torch.randn(steps, B, Hq, 128, generator=gen)).to(cuda_device)
    v = torch.randn(steps, B, Hv, 128, generator=gen).to(torch.bfloat16).to(cuda_device)
    g = (-torch.nn.functional.softplus(torch.randn(steps, B, Hv, generator=gen))).to(cuda_device)
    beta = torch.sigmoid(torch.randn(steps, B, Hv, generator=gen)).to(cuda_device)
    ref_state, ref_out = state0.clone(), torch.empty(steps, B, Hv, 128, device=cuda_device)
    for s in range(steps):
        capi.gdn_decode(ref_state, ref_out[s], q[s], k[s], v[s], g[s], beta[s])
    state, out = state0.clone(), torch.zeros(steps, B, Hv, 128, device=cuda_device)
    graph = GdnDecodeGraph(state, out, q, k, v, g, beta)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(state, ref_state) and torch.equal(out, ref_out)
    # a second replay continues from the updated state, like eight more launches
    for s in range(steps):
        capi.gdn_decode(ref_state, ref_out[s], q[s], k[s], v[s], g[s], beta[s])
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(state, ref_state) and torch.equal(out, ref_out)
