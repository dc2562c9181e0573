"""Full-size runs of the benchmark configurations, checked through properties that do not need a full-size CPU
result.  Needs a GPU.

* rows sampled from the full-size result are compared with the CPU checker (bit-exact forward, 1e-5 gradients),
* spike count == sum of the raster; IAF charge conservation,
* the backward is linear in the upstream gradient,
* a batch shard computed alone equals the same shard of the full run bit for bit, and the time-constant
  gradients of the shards add up to those of the full run (what batch sharding across GPUs relies on).
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests._cases import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-5
DEV = "cuda:0"


def _sample_rows(t_btm, rows_b, rows_m):
    """(B,T,M) device tensor -> [len(rows), T] numpy for the sampled (b, m) pairs."""
    return t_btm.detach()[rows_b, :, rows_m].float().cpu().numpy()


def test_config2_iaf_full_size():
    """IAF on conv feature maps, (32, 300, 32*34*34), 0.4*Poisson(0.1), Heaviside, N(0,1) upstream gradient."""
    from sinabs_exodus_b200 import IntegrateAndFireTM, _lib
    from sinabs_exodus_b200.compat.activation import Heaviside
    B, T, M = 32, 300, 32 * 34 * 34
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.empty(B, T, M, device=DEV)
    for b in range(B):
        x[b] = 0.4 * torch.poisson(torch.full((T, M), 0.1, device=DEV), generator=g)
    x.requires_grad_(True)
    one = torch.ones(1, device=DEV)
    count = torch.zeros(1, dtype=torch.int64, device=DEV)
    fn = Heaviside()
    s, v, v_post = IntegrateAndFireTM.apply(x, one, None, one, None, None, None, fn, None, _lib.RESET_SUBTRACT, count)
    # spike count and charge conservation: sum_t in = v_post_last + theta * sum_t spikes  (alpha = 1, c = theta = 1)
    assert int(count.item()) == int(s.detach().sum(dtype=torch.float64).item())
    lhs = x.detach().sum(1, dtype=torch.float64)
    rhs = v_post.detach().view(B, M).double() + s.detach().sum(1, dtype=torch.float64)
    assert float((lhs - rhs).abs().max()) < 1e-3
    # sampled rows against the CPU checker, bit for bit
    rng = np.random.default_rng(0)
    rb = torch.tensor(rng.integers(0, B, 3000), device=DEV); rm = torch.tensor(rng.integers(0, M, 3000), device=DEV)
    xin = _sample_rows(x.detach(), rb, rm)
    ones = np.ones(3000, np.float32)
    s_ref, v_ref = orc.lif_forward(xin, 0 * ones, ones, ones, ones)
    np.testing.assert_array_equal(_sample_rows(v, rb, rm), v_ref)
    np.testing.assert_array_equal(_sample_rows(s, rb, rm), s_ref)
    # backward: sampled rows against the float64 recurrence; linearity in the upstream gradient
    g1 = torch.empty(B, T, M, device=DEV).normal_(0, 1, generator=g)
    (gi1,) = torch.autograd.grad(s, x, g1, retain_graph=True)
    surr = orc.surrogate_heaviside(v_ref, ones[:, None], 1.0)
    gi64, _ = orc.lif_backward_f64((surr * _sample_rows(g1, rb, rm)).astype(np.float32), surr, np.ones_like(surr), ones, ones)
    assert rel_err(_sample_rows(gi1, rb, rm), gi64) < TOL
    g2 = torch.empty(B, T, M, device=DEV).normal_(0, 1, generator=g)
    (gi2,) = torch.autograd.grad(s, x, g2, retain_graph=True)
    (gi12,) = torch.autograd.grad(s, x, 0.5 * g1 + g2)
    scale = float(gi12.pow(2).mean().sqrt())
    assert float((gi12 - (0.5 * gi1 + gi2)).abs().max()) < 1e-4 * scale
    del gi1, gi2, gi12, g1, g2
    # a batch shard alone == the same shard of the full run
    xs = x.detach()[8:16].contiguous()
    s_sh, v_sh, _ = IntegrateAndFireTM.apply(xs, one, None, one, None, None, None, fn, None, _lib.RESET_SUBTRACT, None)
    assert torch.equal(s_sh, s[8:16]) and torch.equal(v_sh, v[8:16])
    _lib.device_status()


def test_config3_expleak_full_size():
    """ExpLeak, (64, 4000, 512), alpha = exp(-1/50): sampled rows vs the checker, linearity, impulse response."""
    from sinabs_exodus_b200 import LeakyIntegratorTM
    B, T, M = 64, 4000, 512
    g = torch.Generator(device=DEV).manual_seed(2)
    x = torch.empty(B, T, M, device=DEV).normal_(0, 1, generator=g).requires_grad_(True)
    alpha = torch.full((1,), float(np.exp(-1 / 50.0)), device=DEV, requires_grad=True)
    out, v_last = LeakyIntegratorTM.apply(x, alpha, None, None)
    assert torch.equal(v_last.view(B, M), out[:, -1])
    rng = np.random.default_rng(1)
    rb = torch.tensor(rng.integers(0, B, 512), device=DEV); rm = torch.tensor(rng.integers(0, M, 512), device=DEV)
    a_np = np.full(512, alpha.item(), np.float32); z = np.zeros(512, np.float32)
    xin = _sample_rows(x.detach(), rb, rm)
    np.testing.assert_array_equal(_sample_rows(out, rb, rm), orc.leaky_forward(xin, z, a_np))
    go = torch.empty(B, T, M, device=DEV).normal_(0, 1, generator=g)
    gi, ga = torch.autograd.grad(out, (x, alpha), go)
    gi64, ag64 = orc.leaky_backward_f64(_sample_rows(go, rb, rm), a_np, xin, z)
    assert rel_err(_sample_rows(gi, rb, rm), gi64) < TOL
    # impulse response of the whole system: d out[T-1] / d in[0] = alpha^(T-1), read off the input gradient
    e = torch.zeros(B, T, M, device=DEV); e[:, -1] = 1.0
    (gimp,) = torch.autograd.grad(LeakyIntegratorTM.apply(x, alpha.detach(), None, None)[0], x, e)
    want = float(alpha.item()) ** np.arange(T - 1, -1, -1, dtype=np.float64)
    assert rel_err(gimp[3, :, 7].cpu().numpy(), want) < TOL
    assert np.isfinite(ga.item())


def _config4_layer(reset_fn):
    from sinabs_exodus_b200.layers import LIF
    from sinabs_exodus_b200.compat.activation import PeriodicExponential, SingleSpike
    gen = torch.Generator().manual_seed(3)
    tau = 10.0 + 30.0 * torch.rand(1024, generator=gen)
    return LIF(tau_mem=tau, tau_syn=10.0, train_alphas=True, spike_fn=SingleSpike, reset_fn=reset_fn,
               surrogate_grad_fn=PeriodicExponential(), record_states=True).to(DEV)


def _config4_input():
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.empty(128, 500, 1024, device=DEV).normal_(0.2, 0.6, generator=g).requires_grad_(True)
    go = torch.empty(128, 500, 1024, device=DEV).normal_(0, 1, generator=g)
    return x, go


@pytest.mark.parametrize("reset", ["to_zero", "subtract"])
def test_config4_lif_synaptic_full_size(reset):
    """LIF with synaptic stage, per-neuron trainable time constants, SingleSpike, PeriodicExponential on
    (128, 500, 1024) N(0.2, 0.6): with the reset to zero (the fused kernels' reset-to-value form, checked
    against the float64 adjoint and back-propagation through the time-stepped loop in float64) and with the
    subtract reset (checked against the reference's own kernels when they are built)."""
    from oracle.torch_loop import lif_loop
    from sinabs_exodus_b200.compat.activation import MembraneReset, MembraneSubtract, PeriodicExponential
    to_zero = reset == "to_zero"
    B, T, M = 128, 500, 1024
    layer = _config4_layer(MembraneReset(0.0) if to_zero else MembraneSubtract())
    x, go = _config4_input()
    out = layer(x)
    out.backward(go)
    from sinabs_exodus_b200 import _lib
    _lib.device_status()
    assert torch.isfinite(x.grad).all() and torch.isfinite(layer.alpha_mem.grad).all() and torch.isfinite(layer.alpha_syn.grad).all()
    assert abs(layer.firing_rate.item() - out.mean(dtype=torch.float64).item()) < 1e-6
    assert out.max().item() == 1.0

    # ---- sampled rows, forward: both stages bit for bit
    R = 1500
    rng = np.random.default_rng(2)
    rb_np, rm_np = rng.integers(0, B, R), rng.integers(0, M, R)
    rb, rm = torch.tensor(rb_np, device=DEV), torch.tensor(rm_np, device=DEV)
    a_syn = np.full(R, layer.alpha_syn.item(), np.float32)
    a_mem = layer.alpha_mem.detach().cpu().numpy()[rm_np].astype(np.float32)
    s_mem = (np.float32(1.0) - a_mem).astype(np.float32)
    xin = _sample_rows(x.detach(), rb, rm)
    zeros, ones = np.zeros(R, np.float32), np.ones(R, np.float32)
    i_syn = orc.leaky_forward((a_syn[:, None] * xin).astype(np.float32), zeros, a_syn)
    np.testing.assert_array_equal(_sample_rows(layer.recordings["i_syn"].view(B, T, M), rb, rm), i_syn)
    c = zeros if to_zero else ones
    s_ref, v_ref = orc.lif_forward_ext(i_syn, zeros, a_mem, c, ones, None, 1, in_scale=s_mem, reset_to_value=to_zero)
    np.testing.assert_array_equal(_sample_rows(out.detach(), rb, rm), s_ref)
    v_post_ref = np.where(s_ref > 0, np.float32(0.0), v_ref) if to_zero else (v_ref - s_ref).astype(np.float32)
    np.testing.assert_array_equal(_sample_rows(layer.recordings["v_mem"].view(B, T, M), rb, rm), v_post_ref)

    # ---- sampled rows, backward: float64 adjoint of the chain at the forward's own values
    go_rows = _sample_rows(go, rb, rm)
    surr = orc.surrogate_f64("periodic_exponential", v_ref, 1.0, 0.5, 1.0)
    adj = orc.lif_syn_backward_f64(go_rows, v_ref, s_ref, i_syn, xin, surr, zeros, zeros, a_syn, a_syn, s_mem, a_mem, c,
                                   None, to_zero)
    gi_rows = _sample_rows(x.grad, rb, rm)
    assert rel_err(gi_rows, adj["grad_input"]) < TOL

    # ---- the same rows through the time-stepped loop in float64 with autograd (rows as a batch of one-neuron items)
    f64 = lambda a: torch.tensor(np.asarray(a, np.float64))
    xl = f64(xin).reshape(R, T, 1).requires_grad_(True)
    z1 = torch.zeros(R, 1, dtype=torch.float64)
    res = lif_loop(xl, f64(a_mem).reshape(R, 1), z1, torch.ones(1, dtype=torch.float64),
                   None if to_zero else torch.ones(1, dtype=torch.float64), None, PeriodicExponential(), 1,
                   reset_value=0.0 if to_zero else None, alpha_syn=f64(a_syn).reshape(R, 1), i_syn_init=z1,
                   norm_input=True, decay_early=True)
    (res["spikes"] * f64(go_rows).reshape(R, T, 1)).sum().backward()
    v64 = res["v_mem_pre"].detach().reshape(R, T).numpy()
    same = (res["spikes"].detach().reshape(R, T).numpy() == s_ref).all(1) & (np.abs(v64 - 1.0) > 1e-4).all(1)
    assert same.mean() > 0.8, same.mean()
    assert rel_err(v_ref[same], v64[same]) < TOL
    assert rel_err(gi_rows[same], xl.grad.reshape(R, T).numpy()[same]) < TOL

    # ---- subtract reset: the reference's own kernels and Function glue on the sampled rows
    if not to_zero:
        from oracle import ref_gpu
        if ref_gpu.available():
            cu = lambda a: torch.tensor(np.ascontiguousarray(a, np.float32), device=DEV)
            fn = PeriodicExponential()
            a_s, a_m = cu(a_syn), cu(a_mem)
            z, one = cu(zeros), cu(ones)
            pre = (a_s[:, None] * cu(xin)).contiguous()                 # layers/lif.py:194-195 (decay_early)
            i_ref = ref_gpu.leaky_forward(pre, z, a_s)                   # layers/lif.py:190-198
            scaled = ((1.0 - a_m)[:, None] * i_ref).contiguous()         # layers/lif.py:206-209 (norm_input)
            s_k, v_k = ref_gpu.lif_forward(scaled, z, a_m, one, one, None, 1)
            assert torch.equal(s_k, cu(s_ref)) and torch.equal(v_k, cu(v_ref))
            g_scaled, *_ = ref_gpu.integrate_and_fire_backward(cu(go_rows), torch.zeros_like(v_k), v_k, s_k, z, a_m,
                                                               one, one, None, fn, False)
            g_i = ((1.0 - a_m)[:, None] * g_scaled).contiguous()
            g_pre, _, _ = ref_gpu.leaky_backward(g_i, a_s)
            gi_k = (a_s[:, None] * g_pre).cpu().numpy()
            assert rel_err(gi_rows, gi_k) < TOL

    # ---- two batch items alone: the complete per-neuron time-constant gradients against the float64 adjoint
    full_grads = (layer.alpha_mem.grad.clone(), layer.alpha_syn.grad.clone())
    layer.zero_grad(); layer.reset_states()
    x2 = x.detach()[-2:].clone().requires_grad_(True)
    out2 = layer(x2)
    out2.backward(go[-2:])
    assert torch.equal(out2, out[-2:]) and torch.equal(x2.grad, x.grad[-2:])
    nt = lambda t: t.detach().permute(0, 2, 1).reshape(2 * M, T).cpu().numpy()
    am2 = np.tile(layer.alpha_mem.detach().cpu().numpy().astype(np.float32), 2)
    as2 = np.full(2 * M, layer.alpha_syn.item(), np.float32)
    z2, o2 = np.zeros(2 * M, np.float32), np.ones(2 * M, np.float32)
    i2 = nt(layer.recordings["i_syn"].view(2, T, M))
    s2, v2 = orc.lif_forward_ext(i2, z2, am2, z2 if to_zero else o2, o2, None, 1, in_scale=(np.float32(1) - am2), reset_to_value=to_zero)
    np.testing.assert_array_equal(nt(out2), s2)
    adj2 = orc.lif_syn_backward_f64(nt(go[-2:]), v2, s2, i2, nt(x2), orc.surrogate_f64("periodic_exponential", v2, 1.0, 0.5, 1.0),
                                    z2, z2, as2, as2, np.float32(1) - am2, am2, z2 if to_zero else o2, None, to_zero)
    g_am = (adj2["grad_alpha_mem"] - adj2["grad_scale_mem"]).reshape(2, M).sum(0)      # norm_input: scale = 1 - alpha
    g_as = (adj2["grad_alpha_syn"] + adj2["grad_scale_syn"]).sum()                      # decay_early: scale = alpha
    assert rel_err(layer.alpha_mem.grad.cpu().numpy(), g_am) < TOL
    assert abs(layer.alpha_syn.grad.item() - g_as) <= TOL * abs(g_as)

    # ---- the two halves of the batch alone: same spikes and input gradients, time-constant gradients add up
    parts = []
    for lo, hi in ((0, 64), (64, 128)):
        layer.zero_grad(); layer.reset_states()
        xh = x.detach()[lo:hi].clone().requires_grad_(True)
        out_h = layer(xh)
        out_h.backward(go[lo:hi])
        assert torch.equal(out_h, out[lo:hi]) and torch.equal(xh.grad, x.grad[lo:hi])
        parts.append((layer.alpha_mem.grad.clone(), layer.alpha_syn.grad.clone()))
    for k in range(2):
        total = (parts[0][k].double() + parts[1][k].double()).cpu().numpy()
        assert rel_err(full_grads[k].cpu().numpy(), total) < TOL


@pytest.mark.parametrize("norm_input", [True, False], ids=["as_specified", "unnormalised"])
def test_config5_lif_full_size(norm_input):
    """LIF tau_mem=20 (trainable) MultiSpike SingleExponential on (32, 500, 64*64*64) N(0.25, 0.5): 16.8 GB per tensor,
    4 194 304 000 elements, byte offsets beyond 2^32.  Rows are sampled from the last batch items so that the largest
    offsets are the ones checked.  With the layer's default input normalisation (the configuration as specified) the
    potential hovers around 0.25 and hardly any neuron fires; the unnormalised variant of the same layer drives
    every neuron to several spikes per step and exercises the multi-spike path at the same size."""
    from sinabs_exodus_b200 import _lib
    from sinabs_exodus_b200.layers import LIF
    from sinabs_exodus_b200.compat.activation import SingleExponential
    B, T, M = 32, 500, 64 * 64 * 64
    layer = LIF(tau_mem=20.0, surrogate_grad_fn=SingleExponential(), norm_input=norm_input).to(DEV)
    g = torch.Generator(device=DEV).manual_seed(100)
    x = torch.empty(B, T, M, device=DEV).normal_(0.25, 0.5, generator=g).requires_grad_(True)
    go = torch.empty(B, T, M, device=DEV).normal_(0, 1, generator=g)
    out = layer(x)
    out.backward(go)
    _lib.device_status()
    count = int(round(layer.firing_rate.item() * out.numel()))
    total = out.detach().sum(dtype=torch.float64).item()
    assert abs(layer.firing_rate.item() - total / out.numel()) < 1e-6 and abs(count - total) <= 1e-6 * total + 600
    tau_full = layer.tau_mem.grad.clone()
    # sampled rows; three quarters of them from the last two batch items
    R = 3000
    rng = np.random.default_rng(5)
    rb_np = np.where(rng.random(R) < 0.75, rng.integers(B - 2, B, R), rng.integers(0, B, R))
    rm_np = rng.integers(0, M, R); rm_np[:8] = M - 1 - np.arange(8)
    rb_np[:8] = B - 1
    rb, rm = torch.tensor(rb_np, device=DEV), torch.tensor(rm_np, device=DEV)
    xin = _sample_rows(x.detach(), rb, rm)
    with torch.no_grad():
        alpha_t, scale_t = layer._membrane_decay()          # the layer's own float32 values
    a = np.full(R, alpha_t.item(), np.float32)
    sc = np.full(R, scale_t.item() if norm_input else 1.0, np.float32)
    zeros, ones = np.zeros(R, np.float32), np.ones(R, np.float32)
    s_ref, v_ref = orc.lif_forward_ext(xin, zeros, a, ones, ones, None, None, in_scale=sc)
    np.testing.assert_array_equal(_sample_rows(out.detach(), rb, rm), s_ref)
    assert norm_input or ((s_ref > 1).any() and s_ref.mean() > 0.1)
    surr = orc.surrogate_f64("single_exponential", v_ref, 1.0, 0.5, 1.0)
    g_rows = surr * _sample_rows(go, rb, rm).astype(np.float64)
    gi64, _ = orc.lif_backward_f64(g_rows.astype(np.float32), surr.astype(np.float32), np.ones_like(v_ref), a, ones)
    assert rel_err(_sample_rows(x.grad, rb, rm), gi64 * sc[:, None].astype(np.float64)) < TOL
    x_grad_tail = x.grad[-4:].clone()
    out_tail = out.detach()[-4:].clone()
    del out
    x.grad = None
    # the last four batch items alone: identical bits
    layer.zero_grad(); layer.reset_states()
    xs = x.detach()[-4:].clone().requires_grad_(True)
    out_s = layer(xs)
    out_s.backward(go[-4:])
    assert torch.equal(out_s, out_tail) and torch.equal(xs.grad, x_grad_tail)
    del xs, out_s, x_grad_tail, out_tail
    # the two halves alone: their tau gradients add up to the full run's (what the allreduce across ranks computes)
    parts = []
    for lo, hi in ((0, 16), (16, 32)):
        layer.zero_grad(); layer.reset_states()
        xh = x.detach()[lo:hi].requires_grad_(True)
        layer(xh).backward(go[lo:hi])
        parts.append(layer.tau_mem.grad.double().item())
        del xh
    assert abs(tau_full.item() - sum(parts)) <= 2e-5 * abs(sum(parts)), (tau_full.item(), parts)
    _lib.device_status()
