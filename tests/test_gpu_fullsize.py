"""BASELINE-size runs checked through properties that do not need a full-size CPU result.  Needs a GPU.

* rows sampled from the full-size result are compared with the CPU checker (bit-exact forward,
  1e-5 gradients),
* spike count == sum of the raster; IAF charge conservation,
* the backward is linear in the upstream gradient,
* a batch shard computed alone equals the same shard of the full run bit for bit (what batch
  sharding across GPUs relies on).
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


def test_config4_lif_synaptic_full_size():
    """LIF with synaptic stage and per-neuron trainable time constants, (128, 500, 1024): layer-level run,
    sampled rows of both stages vs the checker, batch-shard invariance of the parameter gradients' pieces."""
    from sinabs_exodus_b200.layers import LIF
    from sinabs_exodus_b200.compat.activation import PeriodicExponential, SingleSpike
    B, T, M = 128, 500, 1024
    gen = torch.Generator().manual_seed(3)
    tau = 10.0 + 30.0 * torch.rand(M, generator=gen)
    layer = LIF(tau_mem=tau, tau_syn=10.0, train_alphas=True, spike_fn=SingleSpike,
                surrogate_grad_fn=PeriodicExponential(), record_states=True).to(DEV)
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.empty(B, T, M, device=DEV).normal_(0.2, 0.6, generator=g).requires_grad_(True)
    out = layer(x)
    go = torch.empty(B, T, M, device=DEV).normal_(0, 1, generator=g)
    out.backward(go)
    assert torch.isfinite(x.grad).all() and torch.isfinite(layer.alpha_mem.grad).all() and torch.isfinite(layer.alpha_syn.grad).all()
    assert abs(layer.firing_rate.item() - out.mean(dtype=torch.float64).item()) < 1e-6
    # stage 1 (synapse, decay_early) and stage 2 (spiking, norm_input) on sampled rows
    rng = np.random.default_rng(2)
    rb_np, rm_np = rng.integers(0, B, 1500), rng.integers(0, M, 1500)
    rb, rm = torch.tensor(rb_np, device=DEV), torch.tensor(rm_np, device=DEV)
    a_syn = np.full(1500, layer.alpha_syn.item(), np.float32)
    a_mem = layer.alpha_mem.detach().cpu().numpy()[rm_np].astype(np.float32)
    xin = _sample_rows(x.detach(), rb, rm)
    i_syn = orc.leaky_forward((a_syn[:, None] * xin).astype(np.float32), np.zeros(1500, np.float32), a_syn)
    np.testing.assert_array_equal(_sample_rows(layer.recordings["i_syn"].view(B, T, M), rb, rm), i_syn)
    ones = np.ones(1500, np.float32)
    scaled = ((1.0 - a_mem)[:, None].astype(np.float32) * i_syn).astype(np.float32)
    s_ref, v_ref = orc.lif_forward(scaled, 0 * ones, a_mem, ones, ones, None, 1)
    np.testing.assert_array_equal(_sample_rows(out.detach(), rb, rm), s_ref)
    # half the batch alone gives the same spikes and input gradients for that half
    layer.zero_grad(); layer.reset_states()
    xh = x.detach()[:64].clone().requires_grad_(True)
    out_h = layer(xh)
    out_h.backward(go[:64])
    assert torch.equal(out_h, out[:64]) and torch.equal(xh.grad, x.grad[:64])
