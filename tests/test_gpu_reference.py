"""Ours against the REFERENCE's own CUDA kernels on identical seeded inputs.  Needs a GPU and
``oracle/_ref/libexodus_ref.so`` (the reference kernels compiled for sm_100a by ``oracle/build.py``).

Criteria: v_mem and gradients within 1e-5 relative; spike rasters identical except in rows
whose membrane potential comes within 1e-5 of a multiple of the threshold.
"""
import numpy as np
import pytest
import torch

from oracle import ref_gpu
from tests._cases import lif_case, near_threshold_rows, rel_err

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_gpu.available(), reason="reference kernels not built")]
TOL = 1e-5


def cu(a, grad=False):
    return torch.tensor(np.ascontiguousarray(a, np.float32), device="cuda:0", requires_grad=grad)


@pytest.mark.parametrize("N,T", [(64, 100), (1024, 100), (333, 257), (2000, 64)])
@pytest.mark.parametrize("surrogate", ["single_exp", "heaviside", "periodic"])
@pytest.mark.parametrize("max_spikes", [None, 1])
def test_integrate_and_fire_vs_reference(N, T, surrogate, max_spikes):
    from sinabs_exodus_b200 import IntegrateAndFire
    from sinabs_exodus_b200.compat import activation as sa
    fn = {"single_exp": sa.SingleExponential(), "heaviside": sa.Heaviside(), "periodic": sa.PeriodicExponential()}[surrogate]
    cs = lif_case(N + T, N, T, clamp=True)
    t = {k: cu(v) for k, v in cs.items()}
    rng = np.random.default_rng(N)
    go = cu(rng.standard_normal((N, T)).astype(np.float32))
    gv = cu((0.2 * rng.standard_normal((N, T))).astype(np.float32))

    s_ref, v_ref = ref_gpu.lif_forward(t["inp"], t["v_init"], t["alpha"], t["subtract"], t["theta"], t["theta_low"], max_spikes)
    gi_ref, ga_ref, g0_ref, *_ = ref_gpu.integrate_and_fire_backward(
        go, gv, v_ref, s_ref, t["v_init"], t["alpha"], t["subtract"], t["theta"], t["theta_low"], fn, True)

    inp = t["inp"].clone().requires_grad_(True); alpha = t["alpha"].clone().requires_grad_(True)
    v0 = t["v_init"].clone().requires_grad_(True)
    s, v = IntegrateAndFire.apply(inp, alpha, v0, t["theta"], t["subtract"], t["theta_low"], fn, max_spikes)
    (s * go + v * gv).sum().backward()

    # forward: same roundings as the reference build -> identical bits
    assert torch.equal(v, v_ref)
    assert torch.equal(s, s_ref)
    safe = ~near_threshold_rows(v_ref.cpu().numpy(), cs["theta"])
    assert safe.mean() > 0.9
    assert rel_err(inp.grad.cpu().numpy(), gi_ref.cpu().numpy()) < TOL
    assert rel_err(alpha.grad.cpu().numpy(), ga_ref.cpu().numpy()) < TOL
    assert rel_err(v0.grad.cpu().numpy(), g0_ref.cpu().numpy()) < TOL


@pytest.mark.parametrize("N,T", [(64, 100), (512, 4000), (333, 257)])
def test_leaky_integrator_vs_reference(N, T):
    from sinabs_exodus_b200 import LeakyIntegrator
    rng = np.random.default_rng(N * 3 + T)
    x_np = rng.standard_normal((N, T)).astype(np.float32)
    a_np = rng.uniform(0.5, 1.0, N).astype(np.float32)
    v0_np = rng.standard_normal(N).astype(np.float32)
    go = cu(rng.standard_normal((N, T)).astype(np.float32))
    out_ref = ref_gpu.leaky_forward(cu(x_np), cu(v0_np), cu(a_np))
    gi_ref, ga_ref, g0_ref = ref_gpu.leaky_backward(go, cu(a_np), out_ref, cu(v0_np))
    x, alpha, v0 = cu(x_np, True), cu(a_np, True), cu(v0_np, True)
    out = LeakyIntegrator.apply(x, alpha, v0)
    (out * go).sum().backward()
    assert rel_err(out.detach().cpu().numpy(), out_ref.cpu().numpy()) < TOL
    assert rel_err(x.grad.cpu().numpy(), gi_ref.cpu().numpy()) < TOL
    assert rel_err(alpha.grad.cpu().numpy(), ga_ref.cpu().numpy()) < 2 * TOL
    assert rel_err(v0.grad.cpu().numpy(), g0_ref.cpu().numpy()) < TOL


def test_time_major_forward_matches_reference_bits():
    """The layer-layout kernel on the transposed problem returns the reference's bits."""
    from sinabs_exodus_b200 import IntegrateAndFireTM, _lib
    from sinabs_exodus_b200.compat.activation import SingleExponential
    B, T, M = 4, 120, 96
    cs = lif_case(5, B * M, T, clamp=True)
    t = {k: cu(v) for k, v in cs.items()}
    s_ref, v_ref = ref_gpu.lif_forward(t["inp"], t["v_init"], t["alpha"], t["subtract"], t["theta"], t["theta_low"])
    x = t["inp"].view(B, M, T).permute(0, 2, 1).contiguous()
    s, v, v_post = IntegrateAndFireTM.apply(x, t["alpha"], t["v_init"], t["theta"], t["subtract"], t["theta_low"], None,
                                            SingleExponential(), None, _lib.RESET_SUBTRACT, None)
    assert torch.equal(v.permute(0, 2, 1).reshape(B * M, T), v_ref)
    assert torch.equal(s.permute(0, 2, 1).reshape(B * M, T), s_ref)
