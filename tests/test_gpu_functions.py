"""Autograd Functions and layers on the GPU against the CPU checker.  Needs a GPU."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from oracle.torch_loop import lif_loop
from tests._cases import lif_case, near_threshold_rows, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-5


def cu(a, grad=False):
    return torch.tensor(np.ascontiguousarray(a, np.float32), device="cuda:0", requires_grad=grad)


@pytest.mark.parametrize("surrogate", ["single_exp", "heaviside", "periodic", "callable"])
@pytest.mark.parametrize("backward_var", ["spikes", "vmem", "sum"])
def test_integrate_and_fire_chained(surrogate, backward_var):
    """Three chained calls that carry the state, as reference tests/test_spike_functions.py:69-146."""
    from sinabs_exodus_b200 import IntegrateAndFire
    from sinabs_exodus_b200.compat import activation as sa
    fn_gpu, fn_np = {
        "single_exp": (sa.SingleExponential(), lambda v, th: orc.surrogate_single_exponential(v, th)),
        "heaviside": (sa.Heaviside(0.5), lambda v, th: orc.surrogate_heaviside(v, th, 0.5)),
        "periodic": (sa.PeriodicExponential(), lambda v, th: orc.surrogate_periodic_exponential(v, th)),
        "callable": (lambda v, th: 0.5 / (1.0 + (v - th) ** 2), lambda v, th: (0.5 / (1.0 + (v - th) ** 2)).astype(np.float32)),
    }[surrogate]
    N, T, E = 20, 50, 3
    cs = lif_case(31, N, T * E, clamp=True)
    max_spikes = 2
    inp = cu(cs["inp"], True); alpha = cu(cs["alpha"], True); v0 = cu(cs["v_init"], True)
    theta, c, lo = cu(cs["theta"]), cu(cs["subtract"]), cu(cs["theta_low"])
    v_state = v0
    outs, vms = [], []
    for e in range(E):
        s, vm = IntegrateAndFire.apply(inp[:, e * T:(e + 1) * T].contiguous(), alpha, v_state, theta, c, lo, fn_gpu, max_spikes)
        v_state = vm[:, -1] - c * s[:, -1]
        outs.append(s); vms.append(vm)
    S = torch.cat(outs, 1); V = torch.cat(vms, 1)
    s_ref, v_ref = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"], max_spikes)
    np.testing.assert_array_equal(S.detach().cpu().numpy(), s_ref)
    assert rel_err(V.detach().cpu().numpy(), v_ref) < TOL
    rng = np.random.default_rng(2)
    w_s = rng.random((N, T * E)).astype(np.float32); w_v = rng.random((N, T * E)).astype(np.float32)
    if backward_var == "spikes":
        w_v[:] = 0
    elif backward_var == "vmem":
        w_s[:] = 0
    (S * cu(w_s) + V * cu(w_v)).sum().backward()
    gi, ga, g0 = orc.integrate_and_fire_backward(w_s, w_v, v_ref, s_ref, cs["v_init"], cs["alpha"], cs["subtract"],
                                                 cs["theta"], cs["theta_low"], fn_np, True)
    surr = fn_np(v_ref, cs["theta"][:, None])
    nc = (v_ref > cs["theta_low"][:, None]).astype(np.float32)
    g = (surr * w_s).astype(np.float32) + w_v
    vpost = (v_ref - cs["subtract"][:, None] * s_ref).astype(np.float32)
    gi64, ga64 = orc.lif_backward_f64(g, surr, nc, cs["alpha"], cs["subtract"], vpost, cs["v_init"])
    assert rel_err(inp.grad.cpu().numpy(), gi64) < TOL
    assert rel_err(v0.grad.cpu().numpy(), cs["alpha"] * gi64[:, 0]) < TOL
    # the chained alpha gradient equals the single-call one except for the reference's
    # first-step term, which chained calls apply at every call boundary
    ok = (nc[:, 0] == 1) & (nc[:, T] == 1) & (nc[:, 2 * T] == 1)
    assert rel_err(alpha.grad.cpu().numpy()[ok], ga64[ok]) < TOL


@pytest.mark.parametrize("N,T", [(70, 300), (33, 75), (5, 1), (64, 31), (40, 97), (70, 68), (45, 132), (64, 100), (37, 64), (31, 60)])
@pytest.mark.parametrize("shift", [0, 1, 4, 5, 8])
def test_integrate_and_fire_unaligned_rows(N, T, shift):
    """[N,T] rows that start anywhere inside a 128-byte line (T not a multiple of 32, base pointers
    shifted by a few floats): forward bit-exact, gradients to rounding."""
    from sinabs_exodus_b200 import IntegrateAndFire
    from sinabs_exodus_b200.compat import activation as sa
    cs = lif_case(N * 7 + T, N, T, clamp=True)
    buf = torch.zeros(N * T + shift, device="cuda:0")
    inp = buf[shift:].view(N, T)
    inp.copy_(cu(cs["inp"]))
    assert inp.data_ptr() % 128 == (4 * shift) % 128
    inp.requires_grad_(True)
    alpha = cu(cs["alpha"], True)
    v0, theta, c, lo = cu(cs["v_init"]), cu(cs["theta"]), cu(cs["subtract"]), cu(cs["theta_low"])
    s, vm = IntegrateAndFire.apply(inp, alpha, v0, theta, c, lo, sa.SingleExponential(), None)
    s_ref, v_ref = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"], None)
    np.testing.assert_array_equal(s.detach().cpu().numpy(), s_ref)
    np.testing.assert_array_equal(vm.detach().cpu().numpy(), v_ref)
    rng = np.random.default_rng(N + T)
    w_s = rng.standard_normal((N, T)).astype(np.float32); w_v = rng.standard_normal((N, T)).astype(np.float32)
    gbuf = torch.zeros(N * T + shift, device="cuda:0")
    gs = gbuf[shift:].view(N, T); gs.copy_(cu(w_s))
    torch.autograd.backward([s, vm], [gs, cu(w_v)])
    surr = orc.surrogate_single_exponential(v_ref, cs["theta"][:, None])
    nc = (v_ref > cs["theta_low"][:, None]).astype(np.float32)
    g = (surr * w_s).astype(np.float32) + w_v
    vpost = (v_ref - cs["subtract"][:, None] * s_ref).astype(np.float32)
    gi64, ga64 = orc.lif_backward_f64(g, surr, nc, cs["alpha"], cs["subtract"], vpost, cs["v_init"])
    assert rel_err(inp.grad.cpu().numpy(), gi64) < TOL
    assert rel_err(alpha.grad.cpu().numpy(), ga64) < 2 * TOL


def test_integrate_and_fire_errors():
    from sinabs_exodus_b200 import IntegrateAndFire
    from sinabs_exodus_b200._lib import ExodusLibraryError
    from sinabs_exodus_b200.compat.activation import Heaviside
    N, T = 2, 10
    x = torch.rand(N, T, device="cuda:0"); a = torch.full((N,), 0.9, device="cuda:0"); z = torch.zeros(N, device="cuda:0")
    th = torch.ones(N, device="cuda:0")
    fn = Heaviside(0)
    with pytest.raises(ValueError):
        IntegrateAndFire.apply(x, a, z, th, th, torch.tensor([1.2, 0.0], device="cuda:0"), fn)   # min_v_mem >= threshold
    with pytest.raises(ValueError):
        IntegrateAndFire.apply(x.t(), a, z, th, th, None, fn)                                      # not contiguous
    with pytest.raises(ValueError):
        IntegrateAndFire.apply(x[0], a, z, th, th, None, fn)                                       # not 2D
    with pytest.raises(ValueError):
        IntegrateAndFire.apply(x, a * 2, z, th, th, None, fn)                                      # alpha > 1
    with pytest.raises(ExodusLibraryError):
        IntegrateAndFire.apply(x.cpu(), a.cpu(), z.cpu(), th.cpu(), th.cpu(), None, fn)            # no CPU path
    s, v = IntegrateAndFire.apply(x, a, z, th, None, None, fn)                                     # subtract=None -> threshold
    assert s.shape == v.shape == (N, T)


def test_leaky_integrator_chained():
    """Reference tests/test_leak_functions.py:28-75: forward, input, initial-state and alpha gradients."""
    from sinabs_exodus_b200 import LeakyIntegrator
    N, T, E = 24, 64, 3
    rng = np.random.default_rng(1)
    x_np = rng.random((N, T * E)).astype(np.float32)
    a_np = rng.uniform(0.2, 1.0, N).astype(np.float32); v0_np = rng.standard_normal(N).astype(np.float32)
    w_np = rng.random((N, T * E)).astype(np.float32)
    x, alpha, v0 = cu(x_np, True), cu(a_np, True), cu(v0_np, True)
    state = v0
    outs = []
    for e in range(E):
        o = LeakyIntegrator.apply(x[:, e * T:(e + 1) * T].contiguous(), alpha, state)
        state = o[:, -1].contiguous()
        outs.append(o)
    O = torch.cat(outs, 1)
    (O * cu(w_np)).sum().backward()
    assert rel_err(O.detach().cpu().numpy(), orc.leaky_forward_f64(x_np, v0_np, a_np)) < TOL
    gi64, ag64 = orc.leaky_backward_f64(w_np, a_np, x_np, v0_np)
    assert rel_err(x.grad.cpu().numpy(), gi64) < TOL
    assert rel_err(alpha.grad.cpu().numpy(), ag64) < 2 * TOL
    assert rel_err(v0.grad.cpu().numpy(), a_np * gi64[:, 0]) < TOL
    with pytest.raises(ValueError):
        LeakyIntegrator.apply(x.t(), alpha, v0)


def _loop_ref(layer_kwargs, x_np, **loop_kwargs):
    """CPU ground truth for a layer call: time-stepped loop + autograd."""
    x = torch.tensor(x_np, requires_grad=True)
    res = lif_loop(x, **loop_kwargs)
    return x, res


def test_layer_lif_config1():
    """The CPU-runnable configuration: LIF(tau_mem=20, threshold 1, subtract, MultiSpike, SingleExponential(0.5),
    min_v_mem=-1), all else default (norm_input, trainable tau_mem), input (8,100,128) ~ N(0.3,0.5) seed 0,
    upstream gradient of ones.  Forward bit for bit against the checker; gradients at 1e-5 against the float64
    adjoint at the forward's own values and against back-propagation through the time-stepped loop in float64."""
    from sinabs_exodus_b200.layers import LIF
    from sinabs_exodus_b200.compat.activation import SingleExponential
    torch.manual_seed(0)
    B, T, M = 8, 100, 128
    x_cpu = 0.3 + 0.5 * torch.randn(B, T, M)
    layer = LIF(tau_mem=20.0, spike_threshold=1.0, surrogate_grad_fn=SingleExponential(grad_width=0.5), min_v_mem=-1.0).cuda()
    x = x_cpu.cuda().requires_grad_(True)
    out = layer(x)
    out.sum().backward()
    assert out.shape == x.shape and out.is_contiguous()
    assert "EXODUS" in repr(layer)
    N = B * M
    nt = lambda t: t.detach().cpu().permute(0, 2, 1).reshape(N, T).numpy()
    with torch.no_grad():
        alpha_t, scale_t = layer._membrane_decay()          # the layer's own float32 values
    a = np.full(N, alpha_t.item(), np.float32); sc = np.full(N, scale_t.item(), np.float32)
    one, zero = np.ones(N, np.float32), np.zeros(N, np.float32)
    s_ref, v_ref = orc.lif_forward_ext(nt(x_cpu), zero, a, one, one, -one, None, in_scale=sc)
    np.testing.assert_array_equal(nt(out), s_ref)
    np.testing.assert_allclose(layer.firing_rate.item(), s_ref.mean(dtype=np.float64), rtol=1e-6)
    v_post = (v_ref[:, -1] - s_ref[:, -1]).astype(np.float32)
    np.testing.assert_allclose(layer.v_mem.detach().cpu().numpy().reshape(-1), v_post, rtol=1e-6, atol=1e-7)
    # float64 adjoint at the forward's own v_mem
    surr = orc.surrogate_f64("single_exponential", v_ref, 1.0, 0.5, 1.0)
    nc = (v_ref > -1.0).astype(np.float32)
    gi64, ag64 = orc.lif_backward_f64(surr.astype(np.float32), surr.astype(np.float32), nc, a, one,
                                      (v_ref - s_ref).astype(np.float32), zero)
    assert rel_err(nt(x.grad), gi64 * float(sc[0])) < TOL
    # d/d tau: alpha enters as decay and as norm_input scale 1 - alpha; d alpha / d tau = alpha / tau^2
    sg64 = (gi64 * nt(x_cpu).astype(np.float64)).sum()
    dtau = (ag64.sum() - sg64) * float(a[0]) / 400.0
    dtau_scale = (abs(ag64.sum()) + abs(sg64)) * float(a[0]) / 400.0       # the two parts are formed separately
    assert abs(layer.tau_mem.grad.item() - dtau) <= TOL * dtau_scale, (layer.tau_mem.grad.item(), dtau, dtau_scale)
    # back-propagation through the stepped loop, everything in float64
    f64 = torch.float64
    tau = torch.tensor(20.0, dtype=f64, requires_grad=True)
    xr = x_cpu.to(f64).requires_grad_(True)
    one64 = torch.tensor(1.0, dtype=f64)
    res = lif_loop(xr, torch.exp(-1.0 / tau), torch.zeros(B, M, dtype=f64), one64, one64, -one64,
                   SingleExponential(grad_width=0.5), None, norm_input=True)
    res["spikes"].sum().backward()
    v64 = nt(res["v_mem_pre"])
    safe = ~near_threshold_rows(v64, np.ones(N), rel=1e-4) & (nt(res["spikes"]) == s_ref).all(1)
    assert safe.mean() > 0.9
    assert rel_err(v_ref[safe], v64[safe]) < TOL
    assert rel_err(nt(x.grad)[safe], nt(xr.grad)[safe]) < TOL
    if safe.all():
        assert abs(layer.tau_mem.grad.item() - tau.grad.item()) <= TOL * dtau_scale


def test_layer_lif_sparse_input_long_tau():
    """Sparse input (zero on most steps) and a long membrane time constant: the gradient of tau_mem, whose
    norm_input part the backward rebuilds from the saved membrane potential while 1 - alpha >= 0.01, against the
    float64 adjoint; and the same layer with 1 - alpha < 0.01, which reads the input instead."""
    from sinabs_exodus_b200.layers import LIF
    from sinabs_exodus_b200.compat.activation import SingleExponential
    B, T, M = 16, 300, 256
    N = B * M
    g = torch.Generator().manual_seed(11)
    x_cpu = 20.0 * torch.poisson(torch.full((B, T, M), 0.1), generator=g)
    go_cpu = torch.randn(B, T, M, generator=g)
    nt = lambda t: t.detach().cpu().permute(0, 2, 1).reshape(N, T).numpy()
    for tau0, from_state in ((90.0, True), (150.0, False)):
        layer = LIF(tau_mem=tau0, surrogate_grad_fn=SingleExponential()).cuda()
        x = x_cpu.cuda().requires_grad_(True)
        out = layer(x)
        out.backward(go_cpu.cuda())
        assert bool(getattr(layer, "_scale_nonzero")) == from_state
        with torch.no_grad():
            alpha_t, scale_t = layer._membrane_decay()
        a = np.full(N, alpha_t.item(), np.float32); sc = np.full(N, scale_t.item(), np.float32)
        one, zero = np.ones(N, np.float32), np.zeros(N, np.float32)
        s_ref, v_ref = orc.lif_forward_ext(nt(x_cpu), zero, a, one, one, None, None, in_scale=sc)
        np.testing.assert_array_equal(nt(out), s_ref)
        assert s_ref.sum() > 1000
        surr = orc.surrogate_f64("single_exponential", v_ref, 1.0, 0.5, 1.0)
        g_in = (surr * nt(go_cpu)).astype(np.float32)
        gi64, ag64 = orc.lif_backward_f64(g_in, surr.astype(np.float32), np.ones_like(v_ref), a, one,
                                          (v_ref - s_ref).astype(np.float32), zero)
        assert rel_err(nt(x.grad), gi64 * float(sc[0])) < TOL
        sg64 = (gi64 * nt(x_cpu).astype(np.float64)).sum()
        dtau = (ag64.sum() - sg64) * float(a[0]) / tau0 ** 2
        dtau_scale = (abs(ag64.sum()) + abs(sg64)) * float(a[0]) / tau0 ** 2
        assert abs(layer.tau_mem.grad.item() - dtau) <= TOL * dtau_scale, (tau0, layer.tau_mem.grad.item(), dtau, dtau_scale)


@pytest.mark.parametrize("train_alphas", [False, True])
@pytest.mark.parametrize("norm_input", [False, True])
def test_layer_lif_synaptic_gradients(train_alphas, norm_input):
    """LIF with synaptic stage, per-neuron time constants, non-zero states, two chained calls."""
    from sinabs_exodus_b200.layers import LIF
    from sinabs_exodus_b200.compat.activation import PeriodicExponential, SingleSpike
    B, T, M = 4, 40, 12
    rng = np.random.default_rng(3)
    tau_mem = torch.tensor(rng.uniform(10, 40, M).astype(np.float32))
    x_np = (0.2 + 0.6 * rng.standard_normal((2, B, T, M))).astype(np.float32)
    fn = PeriodicExponential()
    layer = LIF(tau_mem=tau_mem.clone(), tau_syn=10.0, spike_fn=SingleSpike, surrogate_grad_fn=fn, min_v_mem=-1.0,
                train_alphas=train_alphas, norm_input=norm_input, record_states=True).cuda()
    w = torch.tensor(rng.standard_normal((B, T, M)).astype(np.float32))
    xs = [torch.tensor(x_np[e], device="cuda:0", requires_grad=True) for e in range(2)]
    loss = 0
    for e in range(2):
        out = layer(xs[e])
        loss = loss + (out * w.cuda()).sum()
    loss.backward()
    assert set(layer.recordings) == {"i_syn", "v_mem"}

    # ground truth with the same parameterisation, in float64: float32 back-propagation through the
    # stepped loop is itself only good to ~1e-3 for the un-normalised input (large potentials)
    f64 = torch.float64
    tau64 = tau_mem.to(f64)
    if train_alphas:
        p_mem = torch.exp(-1 / tau64).clone().requires_grad_(True); a_mem = p_mem
        p_syn = torch.exp(-1 / torch.tensor(10.0, dtype=f64)).clone().requires_grad_(True); a_syn = p_syn
    else:
        p_mem = tau64.clone().requires_grad_(True); a_mem = torch.exp(-1 / p_mem)
        p_syn = torch.tensor(10.0, dtype=f64, requires_grad=True); a_syn = torch.exp(-1 / p_syn)
    xr = [torch.tensor(x_np[e], dtype=f64, requires_grad=True) for e in range(2)]
    v, i = torch.zeros(B, M, dtype=f64), torch.zeros(B, M, dtype=f64)
    one64 = torch.tensor(1.0, dtype=f64)
    loss_r = 0
    all_v = []
    for e in range(2):
        res = lif_loop(xr[e], a_mem, v, one64, one64, -one64, fn, 1,
                       alpha_syn=a_syn, i_syn_init=i, norm_input=norm_input, decay_early=True)
        v, i = res["v_last"], res["i_last"]
        loss_r = loss_r + (res["spikes"] * w.to(f64)).sum()
        all_v.append(res["v_mem_pre"].detach())
        last = res
    loss_r.backward()
    v_rows = torch.cat(all_v, 1).permute(0, 2, 1).reshape(B * M, -1).numpy()
    safe = ~near_threshold_rows(v_rows, np.ones(B * M, np.float32), rel=1e-4)
    safe_bm = torch.tensor(safe.reshape(B, M))
    for e in range(2):
        g_gpu = xs[e].grad.cpu().permute(0, 2, 1)[safe_bm].numpy()
        g_ref = xr[e].grad.permute(0, 2, 1)[safe_bm].numpy()
        # layer-level check; the 1e-5 parity is checked at kernel level
        assert rel_err(g_gpu, g_ref) < (1e-4 if norm_input else 2e-3)
    if safe.all():
        p_gpu_mem = (layer.alpha_mem if train_alphas else layer.tau_mem).grad.cpu().numpy()
        p_gpu_syn = (layer.alpha_syn if train_alphas else layer.tau_syn).grad.cpu().numpy()
        assert rel_err(p_gpu_mem, p_mem.grad.numpy()) < 1e-3
        assert rel_err(p_gpu_syn, p_syn.grad.numpy()) < 1e-3
    np.testing.assert_allclose(layer.recordings["i_syn"].detach().cpu().numpy(), last["i_syn"].detach().numpy(),
                               rtol=1e-4, atol=1e-5)


def test_layer_iaf_squeeze_and_state():
    """IAFSqueeze on (B*T, C, H, W); state is carried between calls and reset_states clears it."""
    from sinabs_exodus_b200.layers import IAF, IAFSqueeze
    from sinabs_exodus_b200.compat.activation import Heaviside
    B, T, C, H, W = 2, 20, 3, 4, 5
    torch.manual_seed(1)
    x = (0.4 * torch.poisson(torch.full((B, T, C, H, W), 0.4))).cuda()
    sq = IAFSqueeze(batch_size=B, surrogate_grad_fn=Heaviside()).cuda()
    plain = IAF(surrogate_grad_fn=Heaviside()).cuda()
    out_sq = sq(x.reshape(B * T, C, H, W))
    out = plain(x)
    assert out_sq.shape == (B * T, C, H, W)
    torch.testing.assert_close(out_sq.reshape(B, T, C, H, W), out)
    # charge conservation of IAF with subtract = threshold, no clamp: sum(in) = v_post + sum(spikes)
    total_in = x.sum(1)
    torch.testing.assert_close(plain.v_mem + out.sum(1), total_in, rtol=1e-4, atol=1e-4)
    v_before = plain.v_mem.clone()
    out2 = plain(x)
    assert not torch.equal(plain.v_mem, v_before) or torch.equal(out2, out)
    plain.reset_states()
    assert (plain.v_mem == 0).all()
    torch.testing.assert_close(plain(x), out)


@pytest.mark.parametrize("train_alphas", [False, True])
@pytest.mark.parametrize("norm_input", [False, True])
@pytest.mark.parametrize("decay_early", [False, True])
def test_layer_exp_leak(train_alphas, norm_input, decay_early):
    from sinabs_exodus_b200.layers import ExpLeak
    B, T, M = 3, 60, 10
    rng = np.random.default_rng(6)
    x_np = rng.standard_normal((B, T, M)).astype(np.float32)
    w_np = rng.standard_normal((B, T, M)).astype(np.float32)
    layer = ExpLeak(tau_mem=30.0, train_alphas=train_alphas, norm_input=norm_input, decay_early=decay_early).cuda()
    x = torch.tensor(x_np, device="cuda:0", requires_grad=True)
    out = layer(x)
    (out * torch.tensor(w_np, device="cuda:0")).sum().backward()
    if train_alphas:
        p = torch.exp(torch.tensor(-1 / 30.0)).clone().requires_grad_(True); a = p
    else:
        p = torch.tensor(30.0, requires_grad=True); a = torch.exp(-1 / p)
    xr = torch.tensor(x_np, requires_grad=True)
    res = lif_loop(xr, a, torch.zeros(B, M), spiking=False, norm_input=norm_input, decay_early=decay_early)
    (res["v_mem_pre"] * torch.tensor(w_np)).sum().backward()
    assert rel_err(out.detach().cpu().numpy(), res["v_mem_pre"].detach().numpy()) < TOL
    assert rel_err(x.grad.cpu().numpy(), xr.grad.numpy()) < TOL
    g = (layer.alpha_mem if train_alphas else layer.tau_mem).grad.item()
    assert abs(g - p.grad.item()) <= 1e-4 * abs(p.grad.item()) + 1e-6
    # decay_early relation (reference tests/test_exp_leak.py:23-37)
    if decay_early and not norm_input:
        other = ExpLeak(tau_mem=30.0, decay_early=False).cuda()
        want = other(x.detach()) * float(np.exp(-1 / 30.0))
        assert rel_err(out.detach().cpu().numpy(), want.detach().cpu().numpy()) < TOL


def test_layer_exp_leak_firing_rate():
    """`firing_rate` of the non-spiking layer is output.sum() / numel as in the reference layer
    (layers/lif.py:305); here it comes out of the forward kernel, on both kernel routes."""
    from sinabs_exodus_b200.layers import ExpLeak
    for shape in [(3, 50, 40), (2, 3000, 8), (200, 20, 516)]:
        torch.manual_seed(5)
        layer = ExpLeak(tau_mem=20.0).to("cuda:0")
        x = torch.randn(*shape, device="cuda:0") + 0.3
        out = layer(x)
        ref = out.double().sum().item() / out.numel()
        assert abs(layer.firing_rate.item() - ref) <= 1e-5 * (out.double().abs().mean().item() + 1e-12)


def test_layer_exp_leak_long_sequence_uses_scan():
    """Few neurons, long sequence: the layer routes through the time-parallel scan; same results."""
    from sinabs_exodus_b200 import _lib
    from sinabs_exodus_b200.layers import ExpLeak
    B, T, M = 2, 3000, 16
    assert _lib.leaky_scan_workspace_bytes(B, T, M) > 0
    rng = np.random.default_rng(12)
    x_np = rng.standard_normal((B, T, M)).astype(np.float32)
    w_np = rng.standard_normal((B, T, M)).astype(np.float32)
    layer = ExpLeak(tau_mem=torch.tensor(rng.uniform(20, 200, M).astype(np.float32)), norm_input=True).cuda()
    x = torch.tensor(x_np, device="cuda:0", requires_grad=True)
    out = layer(x)
    (out * torch.tensor(w_np, device="cuda:0")).sum().backward()
    # ground truth in float64 from the SAME float32 decay factors (over 3000 steps the result is
    # sensitive to the last bit of alpha); d/d tau follows by the chain rule
    tau = layer.tau_mem.detach().cpu()
    a = torch.exp(-1.0 / tau).double().requires_grad_(True)
    xr = torch.tensor(x_np, dtype=torch.float64, requires_grad=True)
    res = lif_loop(xr, a, torch.zeros(B, M, dtype=torch.float64), spiking=False, norm_input=True, decay_early=False)
    (res["v_mem_pre"] * torch.tensor(w_np, dtype=torch.float64)).sum().backward()
    assert rel_err(out.detach().cpu().numpy(), res["v_mem_pre"].detach().numpy()) < 2 * TOL
    assert rel_err(x.grad.cpu().numpy(), xr.grad.numpy()) < 2 * TOL
    tau_grad = (a.grad * a.detach() / tau.double() ** 2).numpy()
    assert rel_err(layer.tau_mem.grad.cpu().numpy(), tau_grad) < 1e-4
    _lib.device_status()


def test_layer_rejects_cpu_and_bad_config():
    from sinabs_exodus_b200._lib import ExodusLibraryError
    from sinabs_exodus_b200.layers import LIF
    layer = LIF(tau_mem=10.0)
    with pytest.raises(ExodusLibraryError):
        layer(torch.zeros(1, 4, 3))
    with pytest.raises(NotImplementedError):
        LIF(tau_mem=10.0, spike_fn=lambda *a: None)
    bad = LIF(tau_mem=10.0, min_v_mem=2.0).cuda()
    with pytest.raises(ValueError):
        bad(torch.zeros(1, 4, 3, device="cuda:0"))


@pytest.mark.parametrize("B,T,M", [(4, 40, 12), (300, 12, 516), (100, 9, 516)])
@pytest.mark.parametrize("train_alphas", [False, True])
def test_fused_synaptic_layer_equals_two_stage(B, T, M, train_alphas, monkeypatch):
    """The one-kernel LIF+synapse route gives the two-stage route's bits in the forward pass and its
    gradients to rounding (narrow and wide tiles; per-neuron time constants)."""
    import sinabs_exodus_b200.layers.lif as lif_mod
    from sinabs_exodus_b200.layers import LIF
    from sinabs_exodus_b200.compat.activation import SingleExponential
    rng = np.random.default_rng(5)
    tau_mem = torch.tensor(rng.uniform(10, 40, M).astype(np.float32))
    x_np = (0.3 + 0.8 * rng.standard_normal((2, B, T, M))).astype(np.float32)
    w = torch.tensor(rng.standard_normal((B, T, M)).astype(np.float32), device="cuda:0")

    def run(fused):
        if not fused:
            monkeypatch.setattr(lif_mod, "fused_synaptic_eligible", lambda t: False)
        layer = LIF(tau_mem=tau_mem.clone(), tau_syn=8.0, min_v_mem=-1.0, train_alphas=train_alphas,
                    surrogate_grad_fn=SingleExponential(), record_states=True).cuda()
        xs = [torch.tensor(x_np[e], device="cuda:0", requires_grad=True) for e in range(2)]
        outs, loss = [], 0
        for e in range(2):                     # second call starts from the carried states
            out = layer(xs[e])
            outs.append(out)
            loss = loss + (out * w).sum() + 0.1 * layer.recordings["i_syn"].sum()
        loss.backward()
        monkeypatch.undo()
        params = [p.grad.clone() for _, p in sorted(layer.named_parameters())]
        return outs, [x.grad for x in xs], params, layer

    o_f, g_f, p_f, l_f = run(True)
    o_t, g_t, p_t, l_t = run(False)
    for a, b in zip(o_f, o_t):
        assert torch.equal(a, b)
    assert torch.equal(l_f.v_mem, l_t.v_mem) and torch.equal(l_f.i_syn, l_t.i_syn)
    assert torch.equal(l_f.recordings["v_mem"], l_t.recordings["v_mem"])
    for a, b in zip(g_f, g_t):
        assert rel_err(a.cpu().numpy(), b.cpu().numpy()) < TOL
    for a, b in zip(p_f, p_t):
        assert rel_err(a.cpu().numpy(), b.cpu().numpy()) < 1e-4


def test_empty_inputs():
    """No rows or no time steps: nothing is launched, shapes and states pass through."""
    from sinabs_exodus_b200 import IntegrateAndFire, LeakyIntegrator
    from sinabs_exodus_b200.layers import IAF, ExpLeak
    from sinabs_exodus_b200.compat.activation import Heaviside
    dev = "cuda:0"
    a = torch.full((3,), 0.9, device=dev); z = torch.tensor([0.1, -0.2, 0.3], device=dev); th = torch.ones(3, device=dev)
    x0 = torch.zeros(3, 0, device=dev, requires_grad=True)
    s, v = IntegrateAndFire.apply(x0, a, z, th, th, None, Heaviside())
    assert s.shape == v.shape == (3, 0)
    (s.sum() + v.sum()).backward()
    out = LeakyIntegrator.apply(x0, a, z)
    assert out.shape == (3, 0)
    e = torch.zeros(0, device=dev)
    s, v = IntegrateAndFire.apply(torch.zeros(0, 7, device=dev), e, e, e, e, None, Heaviside())
    assert s.shape == (0, 7)
    assert IAF().to(dev)(torch.zeros(2, 0, 5, device=dev)).shape == (2, 0, 5)
    assert ExpLeak(tau_mem=5.0).to(dev)(torch.zeros(0, 4, 5, device=dev)).shape == (0, 4, 5)


def _two_layer_net(M, H):
    from sinabs_exodus_b200.layers import IAF, LIF
    torch.manual_seed(11)
    return torch.nn.Sequential(
        torch.nn.Linear(M, H), LIF(tau_mem=15.0, tau_syn=8.0),
        torch.nn.Linear(H, M), IAF(),
    ).to("cuda:0")


def test_graphed_step_training_matches_eager():
    """A captured forward+backward step replays to the same outputs and gradients as the eager step."""
    from sinabs_exodus_b200 import GraphedStep
    B, T, M, H = 4, 30, 24, 40
    net = _two_layer_net(M, H)
    g = torch.Generator(device="cuda:0").manual_seed(3)
    xs = [torch.randn(B, T, M, device="cuda:0", generator=g) for _ in range(3)]
    gos = [torch.randn(B, T, M, device="cuda:0", generator=g) for _ in range(3)]

    def eager(x, go):
        for m in net.modules():
            if hasattr(m, "reset_states"):
                m.reset_states()
        net.zero_grad(set_to_none=True)
        x = x.clone().requires_grad_(True)
        out = net(x)
        out.backward(go)
        return out.detach().clone(), x.grad.clone(), [p.grad.clone() for p in net.parameters()]

    want = [eager(x, go) for x, go in zip(xs, gos)]
    step = GraphedStep(net, xs[0], gos[0], carry_state=False, input_grad=True)
    for (out_w, gx_w, gp_w), x, go in zip(want, xs, gos):
        out = step(x, go)
        torch.testing.assert_close(out, out_w, rtol=0, atol=0)
        torch.testing.assert_close(step.input_grad, gx_w, rtol=1e-5, atol=1e-6)
        for p, gw in zip(net.parameters(), gp_w):
            torch.testing.assert_close(p.grad, gw, rtol=1e-5, atol=1e-6)


def test_graphed_step_carries_state():
    """carry_state=True: consecutive replays continue from the state the previous one left, as eager calls do."""
    from sinabs_exodus_b200 import GraphedStep
    B, T, M, H = 3, 20, 16, 32
    net = _two_layer_net(M, H)
    g = torch.Generator(device="cuda:0").manual_seed(5)
    chunks = [torch.randn(B, T, M, device="cuda:0", generator=g) for _ in range(4)]
    stateful = [m for m in net.modules() if hasattr(m, "reset_states")]
    with torch.no_grad():
        for m in stateful:
            m.reset_states()
        want = [net(c).clone() for c in chunks]
        v_want = stateful[0].v_mem.clone()
    step = GraphedStep(net, chunks[0], carry_state=True)
    for m in stateful:      # the capture and its warm-up advanced the states: start again from zero
        for name, buf in m.named_buffers(recurse=False):
            buf.zero_()
    for c, w in zip(chunks, want):
        torch.testing.assert_close(step(c), w, rtol=0, atol=0)
    torch.testing.assert_close(stateful[0].v_mem, v_want, rtol=0, atol=0)


def test_graphed_step_truncated_bptt_on_a_container():
    """carry_state=True with an upstream gradient (truncated back-propagation through time) on a Sequential of two
    stateful layers: every replay continues from the detached state of the previous one and gives the outputs and
    parameter gradients of the eager loop that detaches the states between chunks."""
    from sinabs_exodus_b200 import GraphedStep
    B, T, M, H = 3, 20, 16, 32
    net = _two_layer_net(M, H)
    g = torch.Generator(device="cuda:0").manual_seed(9)
    chunks = [torch.randn(B, T, M, device="cuda:0", generator=g) for _ in range(4)]
    gos = [torch.randn(B, T, M, device="cuda:0", generator=g) for _ in range(4)]
    stateful = [m for m in net.modules() if hasattr(m, "reset_states")]
    for m in stateful:
        m.reset_states()

    def eager(c, go):
        for m in stateful:
            m.zero_grad()                      # the layers' own zero_grad detaches their states
        net.zero_grad(set_to_none=True)
        out = net(c)
        out.backward(go)
        return out.detach().clone(), [p.grad.clone() for p in net.parameters()]

    want = [eager(c, go) for c, go in zip(chunks, gos)]
    v_want = stateful[0].v_mem.detach().clone()
    for m in stateful:
        m.zero_grad()                          # nothing of the eager graphs is left alive when the capture starts
    step = GraphedStep(net, chunks[0], gos[0], carry_state=True)      # used to raise in its second warm-up step
    for m in stateful:
        for name, buf in m.named_buffers(recurse=False):
            buf.zero_()
    for (out_w, gp_w), c, go in zip(want, chunks, gos):
        out = step(c, go)
        torch.testing.assert_close(out, out_w, rtol=0, atol=0)
        for p, gw in zip(net.parameters(), gp_w):
            torch.testing.assert_close(p.grad, gw, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(stateful[0].v_mem, v_want, rtol=0, atol=0)


def test_firing_rate_is_differentiable_while_output_is_held():
    """`firing_rate` as the reference sets it (layers/lif.py:305, mean of the output with its graph): a loss on the
    rate reaches the input while the caller holds the output; under no_grad it is a plain number from the kernel's count."""
    from sinabs_exodus_b200.layers import LIF
    torch.manual_seed(4)
    layer = LIF(tau_mem=10.0).to("cuda:0")
    x = (0.5 + torch.randn(3, 25, 16, device="cuda:0")).requires_grad_(True)
    out = layer(x)
    rate = layer.firing_rate
    assert rate.requires_grad
    rate.backward()
    g_rate = x.grad.clone()
    assert g_rate.abs().sum() > 0
    layer.zero_grad(); layer.reset_states(); x.grad = None
    out = layer(x)
    out.mean().backward()
    torch.testing.assert_close(x.grad, g_rate, rtol=1e-5, atol=1e-9)
    with torch.no_grad():
        layer.reset_states()
        out2 = layer(x)
    assert not layer.firing_rate.requires_grad
    torch.testing.assert_close(layer.firing_rate, out2.mean(), rtol=1e-6, atol=0)


def test_layer_recordings_fused_under_no_grad():
    """record_states: with autograd off the recording is a side output of the forward launch; it equals the
    differentiable expression used with autograd on, bit for bit."""
    from sinabs_exodus_b200.layers import LIF
    torch.manual_seed(2)
    x = 0.4 + 0.6 * torch.randn(3, 40, 24, device="cuda:0")
    for kwargs in (dict(tau_mem=15.0, min_v_mem=-0.5), dict(tau_mem=15.0, tau_syn=6.0)):
        a = LIF(record_states=True, **kwargs).to("cuda:0")
        b = LIF(record_states=True, **kwargs).to("cuda:0")
        out_a = a(x.clone().requires_grad_(True))
        with torch.no_grad():
            out_b = b(x)
        torch.testing.assert_close(out_a.detach(), out_b, rtol=0, atol=0)
        torch.testing.assert_close(a.recordings["v_mem"].detach(), b.recordings["v_mem"], rtol=0, atol=0)
        assert a.recordings["v_mem"].requires_grad and not b.recordings["v_mem"].requires_grad


@pytest.mark.parametrize("per_channel_tau", [False, True])
def test_channels_last_input_is_used_where_it_lies(per_channel_tau, monkeypatch):
    """A `channels_last` feature map (what a cuDNN convolution in that memory format hands to the Squeeze layer after
    it, reference layers/iaf.py:96-112): the kernels read it in place -- no copy into row-major order -- and the output
    comes back in `channels_last` memory; values, states and gradients are those of the row-major route."""
    from sinabs_exodus_b200 import _lib
    from sinabs_exodus_b200.layers import LIFSqueeze
    B, T, C, H, W = 2, 12, 8, 5, 6
    torch.manual_seed(5)
    conv = torch.nn.Conv2d(3, C, 3, padding=1).to("cuda:0").to(memory_format=torch.channels_last)
    frames = torch.randn(B * T, 3, H, W, device="cuda:0").to(memory_format=torch.channels_last)
    tau = (10.0 + 20.0 * torch.rand(C, 1, 1)) if per_channel_tau else 15.0
    make = lambda: LIFSqueeze(batch_size=B, tau_mem=tau, min_v_mem=-1.0, record_states=True, norm_input=False).to("cuda:0")
    seen = []
    real = _lib.lif_forward
    monkeypatch.setattr(_lib, "lif_forward", lambda spikes, v_mem, inp, *a, **k: (seen.append(inp.data_ptr()), real(spikes, v_mem, inp, *a, **k))[1])

    def run(layer, as_is):
        conv.zero_grad()
        y = 3.0 * conv(frames)
        assert y.is_contiguous(memory_format=torch.channels_last) and not y.is_contiguous()
        y_in = y if as_is else y.contiguous()
        outs = []
        for _ in range(2):                       # the second call starts from the carried state
            outs.append(layer(y_in))
        w = torch.arange(outs[0].numel(), device="cuda:0", dtype=torch.float32).reshape(outs[0].shape).cos()
        ((outs[0] + outs[1]) * w).sum().backward()
        grads = [p.grad.clone() for p in list(conv.parameters()) + list(layer.parameters())]
        return y, outs, grads

    a, b = make(), make()
    y, outs_a, grads_a = run(a, True)
    assert seen[0] == y.data_ptr()                                    # the kernel got the convolution's own memory
    assert outs_a[0].is_contiguous(memory_format=torch.channels_last)
    _, outs_b, grads_b = run(b, False)
    for oa, ob in zip(outs_a, outs_b):
        torch.testing.assert_close(oa, ob, rtol=0, atol=0)
    torch.testing.assert_close(a.v_mem, b.v_mem, rtol=0, atol=0)
    torch.testing.assert_close(a.recordings["v_mem"], b.recordings["v_mem"], rtol=0, atol=0)
    assert outs_a[0].sum() > 0
    for ga, gb in zip(grads_a, grads_b):
        torch.testing.assert_close(ga, gb, rtol=1e-4, atol=1e-5)
