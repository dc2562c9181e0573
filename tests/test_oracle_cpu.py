"""The CPU checker against known answers and against itself (no GPU)."""
import glob
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests._cases import lif_case, rel_err

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_notebook_known_answer():
    """IAF, theta=0.9, c=0.8, boxcar surrogate 1/theta: d a_T / d I_{T-n} = 1.111.. * 0.111..^n
    (worked example of the reference's Gradient_analysis.ipynb, cells 1-4)."""
    T = 5
    theta = np.array([0.9], np.float32); c = np.array([0.8], np.float32); alpha = np.ones(1, np.float32)
    surr = np.full((1, T), 1.0 / 0.9, np.float32)
    go = np.zeros((1, T), np.float32); go[0, -1] = 1.0       # gradient of the last output only
    g = surr * go
    gi = orc.lif_backward(g, surr, np.ones_like(surr), alpha, alpha * c)
    want = np.array([(1 / 0.9) * (1 - 0.8 / 0.9) ** n for n in range(T - 1, -1, -1)])
    np.testing.assert_allclose(gi[0], want, rtol=1e-5)
    np.testing.assert_allclose(want, [0.00017, 0.00152, 0.01372, 0.12346, 1.11111], atol=5e-6)


def test_leaky_impulse_response():
    """v_T = alpha^(T-1) for a unit impulse at t=0 (reference tests/test_exp_leak.py:53-75)."""
    T = 50
    alpha = np.array([np.exp(-1 / 10.0)], np.float32)
    x = np.zeros((1, T), np.float32); x[0, 0] = 1.0
    out = orc.leaky_forward(x, np.zeros(1, np.float32), alpha)
    np.testing.assert_allclose(out[0, -1], float(alpha[0]) ** (T - 1), rtol=1e-5)


def test_forward_hand_computed():
    """Three steps by hand: subtract reset uses the previous count before the decay."""
    x = np.array([[1.5, 0.2, 2.4]], np.float32)
    one = np.ones(1, np.float32)
    s, v = orc.lif_forward(x, np.zeros(1, np.float32), 0.5 * one, one, one)
    # t0: v=1.5 -> 1 spike; t1: (1.5-1)*.5+.2=.45 -> 0; t2: .45*.5+2.4=2.625 -> 2 spikes
    np.testing.assert_array_equal(s, [[1, 0, 2]])
    np.testing.assert_allclose(v, [[1.5, 0.45, 2.625]], rtol=1e-6)
    s1, _ = orc.lif_forward(x, np.zeros(1, np.float32), 0.5 * one, one, one, max_spikes=1)
    np.testing.assert_array_equal(s1, [[1, 0, 1]])
    # lower bound
    xl = np.array([[-3.0, 0.5]], np.float32)
    _, vl = orc.lif_forward(xl, np.zeros(1, np.float32), one, one, one, theta_low=-one)
    np.testing.assert_allclose(vl, [[-1.0, -0.5]])


@pytest.mark.parametrize("clamp", [False, True])
def test_double_loop_equals_reverse_recurrence(clamp):
    """The reference's O(T^2) sum and the O(T) reverse recurrence are the same function;
    same for the alpha gradient and its adjoint form (including the first-step term)."""
    cs = lif_case(11, N=37, T=41, clamp=clamp)
    s, v = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"])
    rng = np.random.default_rng(5)
    go = rng.standard_normal(v.shape).astype(np.float32)
    surr = orc.surrogate_single_exponential(v, cs["theta"][:, None])
    nc = (v > cs["theta_low"][:, None]).astype(np.float32) if clamp else np.ones_like(v)
    g = surr * go
    gi32 = orc.lif_backward(g, surr, nc, cs["alpha"], cs["alpha"] * cs["subtract"])
    vpost = (v - cs["subtract"][:, None] * s).astype(np.float32)
    ag32 = orc.lif_backward_alpha(g, vpost, cs["v_init"], surr, nc, cs["alpha"], cs["subtract"])
    gi64, ag64 = orc.lif_backward_f64(g, surr, nc, cs["alpha"], cs["subtract"], vpost, cs["v_init"])
    assert rel_err(gi32, gi64) < 1e-5
    assert rel_err(ag32, ag64) < 1e-5
    if clamp:
        assert (nc[:, 0] == 0).any() or True   # the first-step term is exercised when a row starts clipped


def test_first_step_clip_term():
    """A row whose first step is clipped and whose v_init is non-zero: the reference carries
    v_init into step 1 ungated (cuda/lif_kernels.h:219-238); the f64 form must reproduce it."""
    N, T = 4, 6
    inp = np.full((N, T), 0.3, np.float32); inp[:, 0] = -5.0
    alpha = np.full(N, 0.9, np.float32); theta = np.ones(N, np.float32); c = theta.copy()
    lo = np.full(N, -1.0, np.float32); v0 = np.array([0.4, -0.2, 0.0, 0.7], np.float32)
    s, v = orc.lif_forward(inp, v0, alpha, c, theta, lo)
    assert (v[:, 0] == -1.0).all()
    surr = orc.surrogate_single_exponential(v, theta[:, None])
    nc = (v > lo[:, None]).astype(np.float32)
    go = np.ones_like(v)
    g = surr * go
    vpost = (v - c[:, None] * s).astype(np.float32)
    ag32 = orc.lif_backward_alpha(g, vpost, v0, surr, nc, alpha, c)
    _, ag64 = orc.lif_backward_f64(g, surr, nc, alpha, c, vpost, v0)
    assert rel_err(ag32, ag64) < 1e-5
    # and the term is really there: with v_init = 0 the result differs
    ag0 = orc.lif_backward_alpha(g, vpost, np.zeros(N, np.float32), surr, nc, alpha, c)
    assert np.abs(ag32 - ag0)[[0, 1, 3]].min() > 1e-4


def test_leaky_backward_forms():
    rng = np.random.default_rng(3)
    N, T = 19, 67
    x = rng.standard_normal((N, T)).astype(np.float32)
    go = rng.standard_normal((N, T)).astype(np.float32)
    alpha = rng.uniform(0.3, 1.0, N).astype(np.float32); v0 = rng.standard_normal(N).astype(np.float32)
    out = orc.leaky_forward(x, v0, alpha)
    gi = orc.leaky_backward(go, alpha)
    ag = orc.leaky_backward_alpha(go, out, v0, alpha)
    gi64, ag64 = orc.leaky_backward_f64(go, alpha, x, v0)
    assert rel_err(out, orc.leaky_forward_f64(x, v0, alpha)) < 1e-5
    assert rel_err(gi, gi64) < 1e-5
    assert rel_err(ag, ag64) < 1e-5


def test_bptt_loop_matches_exodus_backward():
    """Back-propagation through the time-stepped PyTorch loop gives the gradients of the
    single-pass EXODUS backward (input, initial state, alpha)."""
    import torch
    from oracle.torch_loop import lif_loop
    from sinabs_exodus_b200.compat.activation import SingleExponential

    cs = lif_case(21, N=6, T=25, clamp=True)
    x = torch.tensor(cs["inp"]).reshape(1, 6, 25).permute(0, 2, 1).contiguous().requires_grad_(True)  # (B=1,T,M)
    alpha = torch.tensor(cs["alpha"], requires_grad=True)
    v0 = torch.tensor(cs["v_init"]).reshape(1, 6).requires_grad_(True)
    fn = SingleExponential()
    res = lif_loop(x, alpha, v0, torch.tensor(cs["theta"]), torch.tensor(cs["subtract"]),
                   torch.tensor(cs["theta_low"]), fn, None)
    w = torch.tensor(np.random.default_rng(0).standard_normal((1, 25, 6)).astype(np.float32))
    (res["spikes"] * w).sum().backward()
    s, v = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"])
    np.testing.assert_array_equal(res["spikes"][0].T.detach().numpy(), s)
    go = w[0].T.numpy()
    gi, ga, g0 = orc.integrate_and_fire_backward(
        go, np.zeros_like(go), v, s, cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"],
        lambda vv, th: orc.surrogate_single_exponential(vv, th), True)
    assert rel_err(gi, x.grad[0].T.numpy()) < 1e-4
    assert rel_err(g0, v0.grad[0].numpy()) < 1e-4
    # rows whose first step is clipped carry the reference's extra term; compare the others
    ok = v[:, 0] > cs["theta_low"]
    assert rel_err(ga[ok], alpha.grad.numpy()[ok]) < 1e-4


def test_fma_association_matters():
    """The two builds of the checker differ in the last bit somewhere: the association is observable."""
    cs = lif_case(2, N=64, T=200)
    _, v_fma = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], fma=True)
    _, v_mul = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], fma=False)
    assert rel_err(v_fma, v_mul) < 1e-4
    assert (v_fma != v_mul).any()


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "*.npz"))) or [None])
def test_golden_vectors(path):
    """Outputs of the reference's own kernels (sm_100a build, run on a B200) pin the checker."""
    if path is None:
        pytest.skip("no golden vectors committed yet")
    g = dict(np.load(path))
    kind = str(g["kind"])
    if kind == "lif":
        lo = g["theta_low"] if g["apply_theta_low"] else None
        ms = None if int(g["max_spikes"]) < 0 else int(g["max_spikes"])
        s, v = orc.lif_forward(g["inp"], g["v_init"], g["alpha"], g["subtract"], g["theta"], lo, ms)
        np.testing.assert_array_equal(s, g["ref_spikes"])
        np.testing.assert_array_equal(v, g["ref_v_mem"])
        gi = orc.lif_backward(g["g"], g["surr"], g["not_clipped"], g["alpha"], g["alpha"] * g["subtract"])
        assert rel_err(gi, g["ref_grad_input"]) < 1e-6
        ag = orc.lif_backward_alpha(g["g"], g["v_post"], g["v_init"], g["surr"], g["not_clipped"], g["alpha"],
                                    g["subtract"])
        assert rel_err(ag, g["ref_grad_alpha"]) < 1e-6
    else:
        out = orc.leaky_forward(g["inp"], g["v_init"], g["alpha"])
        np.testing.assert_array_equal(out, g["ref_out"])
        np.testing.assert_array_equal(orc.leaky_backward(g["go"], g["alpha"]), g["ref_grad_input"])
        ag = orc.leaky_backward_alpha(g["go"], g["ref_out"], g["v_init"], g["alpha"])
        assert rel_err(ag, g["ref_grad_alpha"]) < 1e-6


def test_forward_ext_reduces_to_reference_forward():
    """Without a scale and with the subtract reset the extended forward is the reference forward bit for bit; with a
    scale it equals the reference forward on the pre-multiplied input (a separate rounded product)."""
    cs = lif_case(5, N=40, T=60, clamp=True)
    s0, v0 = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"], 3)
    s1, v1 = orc.lif_forward_ext(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"], 3)
    np.testing.assert_array_equal(s0, s1); np.testing.assert_array_equal(v0, v1)
    sc = np.random.default_rng(1).uniform(0.1, 2.0, 40).astype(np.float32)
    s2, v2 = orc.lif_forward_ext(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], None, None, in_scale=sc)
    s3, v3 = orc.lif_forward((sc[:, None] * cs["inp"]).astype(np.float32), cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"])
    np.testing.assert_array_equal(s2, s3); np.testing.assert_array_equal(v2, v3)


def test_forward_ext_reset_to_value_by_hand():
    x = np.array([[1.5, 0.2, 2.4, 0.1]], np.float32)
    one = np.ones(1, np.float32)
    s, v = orc.lif_forward_ext(x, np.zeros(1, np.float32), 0.5 * one, 0.25 * one, one, reset_to_value=True)
    # t0: 1.5 -> spike, reset to .25; t1: .25*.5+.2=.325; t2: .325*.5+2.4=2.5625 -> 2 spikes, reset; t3: .25*.5+.1
    np.testing.assert_array_equal(s, [[1, 0, 2, 0]])
    np.testing.assert_allclose(v, [[1.5, 0.325, 2.5625, 0.225]], rtol=1e-6)


@pytest.mark.parametrize("reset_to_value", [False, True])
@pytest.mark.parametrize("surrogate", ["single_exponential", "heaviside", "periodic_exponential"])
def test_synaptic_adjoint_f64_equals_bptt(reset_to_value, surrogate):
    """The float64 adjoint of the two-stage layer chain (synapse -> scale -> spiking membrane) equals
    back-propagation through the time-stepped loop in float64: input gradient, both initial states and all four
    parameter gradients, with gradients arriving on spikes, v_mem, i_syn and on both final states."""
    import torch
    from oracle.torch_loop import lif_loop
    from sinabs_exodus_b200.compat import activation as sa

    fn, p0 = {"single_exponential": (sa.SingleExponential(0.7, 1.3), 0.7), "heaviside": (sa.Heaviside(0.6), 0.6),
              "periodic_exponential": (sa.PeriodicExponential(0.4, 0.9), 0.4)}[surrogate]
    p1 = getattr(fn, "grad_scale", 1.0)
    rng = np.random.default_rng(17)
    B, T, M = 2, 40, 7
    dt = torch.float64
    x = torch.tensor(1.5 + 4.0 * rng.standard_normal((B, T, M)), dtype=dt, requires_grad=True)
    a_mem = torch.tensor(rng.uniform(0.4, 0.9, M), dtype=dt, requires_grad=True)
    a_syn = torch.tensor(rng.uniform(0.5, 0.95, M), dtype=dt, requires_grad=True)
    v0 = torch.tensor(rng.uniform(-0.3, 0.3, (B, M)), dtype=dt, requires_grad=True)
    i0 = torch.tensor(rng.uniform(-0.3, 0.3, (B, M)), dtype=dt, requires_grad=True)
    theta = torch.tensor(rng.uniform(0.5, 1.1, M), dtype=dt)
    c = torch.tensor(rng.uniform(0.2, 0.5, M), dtype=dt)
    lo = torch.tensor(-rng.uniform(0.1, 0.4, M), dtype=dt)
    res = lif_loop(x, a_mem, v0, theta, c, lo, fn, 2, reset_value=None, alpha_syn=a_syn, i_syn_init=i0,
                   norm_input=True, decay_early=True) if not reset_to_value else None
    if reset_to_value:
        # per-neuron reset values are not an option of the loop: use one value
        c = torch.full((M,), 0.15, dtype=dt)
        res = lif_loop(x, a_mem, v0, theta, None, lo, fn, 2, reset_value=0.15, alpha_syn=a_syn, i_syn_init=i0,
                       norm_input=True, decay_early=True)
    w = {k: torch.tensor(rng.standard_normal((B, T, M)), dtype=dt) for k in ("s", "v", "i")}
    wl = {k: torch.tensor(rng.standard_normal((B, M)), dtype=dt) for k in ("v", "i")}
    loss = ((res["spikes"] * w["s"]).sum() + (res["v_mem_pre"] * w["v"]).sum() + (res["i_syn"] * w["i"]).sum()
            + (res["v_last"] * wl["v"]).sum() + (res["i_last"] * wl["i"]).sum())
    loss.backward()

    nt = lambda t: t.detach().permute(0, 2, 1).reshape(B * M, T).numpy()       # (B,T,M) -> [N,T]
    per_n = lambda t: np.tile(t.detach().numpy(), B)                           # (M,) -> (N,)
    v = nt(res["v_mem_pre"])
    surr = orc.surrogate_f64(surrogate, v, per_n(theta)[:, None], p0, p1)
    got = orc.lif_syn_backward_f64(
        nt(w["s"]), v, nt(res["spikes"]), nt(res["i_syn"]), nt(x), surr, v0.detach().reshape(-1).numpy(),
        i0.detach().reshape(-1).numpy(), per_n(a_syn), per_n(a_syn), per_n(1.0 - a_mem), per_n(a_mem), per_n(c),
        per_n(lo), reset_to_value, grad_v_mem=nt(w["v"]), grad_v_last=wl["v"].reshape(-1).numpy(),
        grad_i_syn=nt(w["i"]), grad_i_last=wl["i"].reshape(-1).numpy())
    assert (nt(res["spikes"]) > 1).any() and (v <= per_n(lo)[:, None]).any()
    tol = 1e-10
    assert rel_err(got["grad_input"], nt(x.grad)) < tol
    assert rel_err(got["grad_v_init"], v0.grad.reshape(-1).numpy()) < tol
    assert rel_err(got["grad_i_init"], i0.grad.reshape(-1).numpy()) < tol
    # parameters: alpha_mem enters as decay and, through norm_input, as scale 1 - alpha_mem; alpha_syn as decay
    # and, through decay_early, as the input scale.  Rows whose first step is clipped carry the reference's extra
    # first-step term, which back-propagation through the loop does not have: leave those neurons out.
    first_clipped = (v[:, 0] <= per_n(lo)).reshape(B, M).any(0)
    ok = ~first_clipped
    g_am = (got["grad_alpha_mem"] - got["grad_scale_mem"]).reshape(B, M).sum(0)
    g_as = (got["grad_alpha_syn"] + got["grad_scale_syn"]).reshape(B, M).sum(0)
    assert ok.any()
    assert rel_err(g_am[ok], a_mem.grad.numpy()[ok]) < tol
    assert rel_err(g_as, a_syn.grad.numpy()) < tol
