"""Decay and scale derived inside the kernels (EXB_PARAM_IS_TAU, EXB_SCALE_*) and parameter gradients reduced inside
the backward kernels (acc_decay), against the same calls with explicit alpha / scale tensors and per-instance
outputs.  Needs a GPU."""
import numpy as np
import pytest
import torch

from sinabs_exodus_b200 import _lib
from tests._cases import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-5
L = _lib.LAYOUT_BTM


def _param(rng, lo, hi, mode, B, M):
    n = {_lib.PARAM_SCALAR: 1, _lib.PARAM_PER_M: M, _lib.PARAM_PER_N: B * M}[mode]
    return torch.tensor(rng.uniform(lo, hi, n).astype(np.float32), device=DEV)


def _reduce(per_instance, mode, B, M):
    g = per_instance.double()
    if mode == _lib.PARAM_SCALAR:
        return g.sum().reshape(1)
    if mode == _lib.PARAM_PER_M:
        return g.view(B, M).sum(0)
    return g


def _fold(ga, gs, tau, alpha, scale_flags):
    """float64 chain rule: gradient w.r.t. tau from the gradients w.r.t. alpha and the derived scale."""
    a = alpha.double()
    g = ga.clone()
    om, ta = scale_flags & _lib.SCALE_ONE_MINUS_ALPHA, scale_flags & _lib.SCALE_TIMES_ALPHA
    if om and ta:
        g = g + (1 - 2 * a) * gs
    elif om:
        g = g - gs
    elif ta:
        g = g + gs
    return g * a / tau.double() ** 2


SHAPES = [(3, 37, 64), (5, 23, 132), (37, 9, 4096)]
MODES = [_lib.PARAM_SCALAR, _lib.PARAM_PER_M, _lib.PARAM_PER_N]


@pytest.mark.parametrize("B,T,M", SHAPES)
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("scale_flags", [0, _lib.SCALE_ONE_MINUS_ALPHA])
def test_lif_tau_and_derived_scale(B, T, M, mode, scale_flags):
    rng = np.random.default_rng(B * 100 + M + mode)
    N = B * M
    x = torch.tensor((0.5 + 1.5 * rng.standard_normal((B, T, M))).astype(np.float32), device=DEV)
    go = torch.tensor(rng.standard_normal((B, T, M)).astype(np.float32), device=DEV)
    tau = _param(rng, 3.0, 30.0, mode, B, M)
    alpha = torch.exp(-torch.reciprocal(tau))
    scale = (1.0 - alpha) if scale_flags else None
    theta = torch.ones(1, device=DEV)
    v0 = torch.tensor(rng.uniform(-0.3, 0.3, N).astype(np.float32), device=DEV)
    none = (None, 0)

    def forward(a_spec, s_spec):
        s = torch.empty_like(x); v = torch.empty_like(x); vp = torch.empty(N, device=DEV)
        _lib.lif_forward(s, v, x, v0, s_spec, a_spec, none, (theta, 0), none, None, _lib.RESET_SUBTRACT, vp, None, B, T, M, L)
        return s, v, vp

    s_ref, v_ref, vp_ref = forward((alpha, mode), (scale, mode) if scale is not None else none)
    s, v, vp = forward((tau, mode | _lib.PARAM_IS_TAU), (None, mode | scale_flags) if scale_flags else none)
    assert torch.equal(s, s_ref) and torch.equal(v, v_ref) and torch.equal(vp, vp_ref)
    assert s.sum() > 0

    def backward(a_spec, s_spec, per_instance, acc, inp):
        gi = torch.empty_like(x); g0 = torch.empty(N, device=DEV)
        ga = torch.empty(N, device=DEV) if per_instance else None
        gs = torch.empty(N, device=DEV) if (per_instance and s_spec is not none) else None
        ok = _lib.lif_backward(gi, ga, g0, gs, go, None, None, v_ref, None, v0, inp, s_spec, a_spec, none, (theta, 0), none,
                               None, _lib.RESET_SUBTRACT, _lib.SURR_SINGLE_EXPONENTIAL, 0.5, 1.0, B, T, M, L, acc_decay=acc)
        assert ok
        return gi, ga, g0, gs

    for from_state in (False, True):
        inp = None if from_state else x
        gi_ref, ga_ref, g0_ref, gs_ref = backward((alpha, mode), (scale, mode) if scale is not None else none, True, None, inp)
        want = _fold(_reduce(ga_ref, mode, B, M), _reduce(gs_ref, mode, B, M) if gs_ref is not None else 0.0, tau, alpha, scale_flags)
        acc = torch.zeros(tau.numel(), dtype=torch.float64, device=DEV)
        gi, _, g0, _ = backward((tau, mode | _lib.PARAM_IS_TAU), (None, mode | scale_flags) if scale_flags else none, False, acc, inp)
        assert torch.equal(gi, gi_ref) and torch.equal(g0, g0_ref)
        assert rel_err(acc.cpu().numpy(), want.cpu().numpy()) < TOL
        out = torch.empty(tau.numel(), device=DEV)
        _lib.acc_finish(out, acc)
        assert torch.equal(acc, torch.zeros_like(acc))
        assert rel_err(out.cpu().numpy(), want.cpu().numpy()) < TOL


@pytest.mark.parametrize("B,T,M", [(3, 37, 64), (2, 4000, 128), (37, 9, 4096)])
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("scale_flags", [0, _lib.SCALE_ONE_MINUS_ALPHA, _lib.SCALE_TIMES_ALPHA,
                                         _lib.SCALE_ONE_MINUS_ALPHA | _lib.SCALE_TIMES_ALPHA])
def test_leaky_tau_and_derived_scale(B, T, M, mode, scale_flags):
    """The leaky integrator, plain and time-parallel (the long shape): derived alpha and scale bit for bit; the
    accumulated tau gradient against the folded per-instance gradients."""
    rng = np.random.default_rng(B + T + M + mode + scale_flags)
    N = B * M
    x = torch.tensor(rng.standard_normal((B, T, M)).astype(np.float32), device=DEV)
    go = torch.tensor(rng.standard_normal((B, T, M)).astype(np.float32), device=DEV)
    tau = _param(rng, 5.0, 60.0, mode, B, M)
    alpha = torch.exp(-torch.reciprocal(tau))
    scale = None
    if scale_flags & _lib.SCALE_ONE_MINUS_ALPHA:
        scale = 1.0 - alpha
    if scale_flags & _lib.SCALE_TIMES_ALPHA:
        scale = alpha.clone() if scale is None else scale * alpha
    v0 = torch.tensor(rng.standard_normal(N).astype(np.float32), device=DEV)
    none = (None, 0)
    s_ref = (scale, mode) if scale is not None else none
    s_new = (None, mode | scale_flags) if scale_flags else none
    nbytes = _lib.leaky_scan_workspace_bytes(B, T, M)
    ws = torch.zeros((nbytes + 3) // 4, dtype=torch.int32, device=DEV) if nbytes else None

    def forward(a_spec, s_spec, clean):
        out = torch.empty_like(x); vl = torch.empty(N, device=DEV)
        if ws is not None:
            _lib.leaky_forward_scan(out, x, v0, a_spec, s_spec, vl, ws, B, T, M, clean=clean)
        else:
            _lib.leaky_forward(out, x, v0, a_spec, s_spec, vl, B, T, M, L)
        return out, vl

    out_ref, vl_ref = forward((alpha, mode), s_ref, False)
    out, vl = forward((tau, mode | _lib.PARAM_IS_TAU), s_new, True)      # the workspace was left clean by the call before
    assert torch.equal(out, out_ref) and torch.equal(vl, vl_ref)

    def backward(a_spec, s_spec, per_instance, acc, clean):
        gi = torch.empty_like(x); g0 = torch.empty(N, device=DEV)
        ga = torch.empty(N, device=DEV) if per_instance else None
        gs = torch.empty(N, device=DEV) if (per_instance and s_spec is not none) else None
        if ws is not None:
            _lib.leaky_backward_scan(gi, ga, g0, gs, go, None, out_ref, x, v0, a_spec, s_spec, ws, B, T, M, acc_decay=acc, clean=clean)
        else:
            assert _lib.leaky_backward(gi, ga, g0, gs, go, None, out_ref, x, v0, a_spec, s_spec, B, T, M, L, acc_decay=acc)
        return gi, ga, g0, gs

    gi_ref, ga_ref, g0_ref, gs_ref = backward((alpha, mode), s_ref, True, None, True)
    want = _fold(_reduce(ga_ref, mode, B, M), _reduce(gs_ref, mode, B, M) if gs_ref is not None else 0.0, tau, alpha, scale_flags)
    acc = torch.zeros(tau.numel(), dtype=torch.float64, device=DEV)
    gi, _, g0, _ = backward((tau, mode | _lib.PARAM_IS_TAU), s_new, False, acc, True)
    assert torch.equal(gi, gi_ref) and torch.equal(g0, g0_ref)
    assert rel_err(acc.cpu().numpy(), want.cpu().numpy()) < TOL
    if ws is not None:
        assert int(ws[:16 + 64].abs().sum()) == 0                          # counters and flags back to zero


def test_accumulator_needs_an_eligible_shape():
    """Neurons not a multiple of 4: the reducing kernels do not apply; the binding reports it and launches nothing."""
    B, T, M = 2, 10, 30
    x = torch.randn(B, T, M, device=DEV); v = torch.randn(B, T, M, device=DEV)
    alpha = torch.full((1,), 0.9, device=DEV); theta = torch.ones(1, device=DEV)
    acc = torch.zeros(1, dtype=torch.float64, device=DEV)
    gi = torch.empty_like(x)
    ok = _lib.lif_backward(gi, None, None, None, x, None, None, v, None, None, None, (None, 0), (alpha, 0), (None, 0),
                           (theta, 0), (None, 0), None, _lib.RESET_SUBTRACT, _lib.SURR_HEAVISIDE, 1.0, 0.0, B, T, M, L,
                           acc_decay=acc)
    assert ok is False and acc.item() == 0.0
    ok = _lib.leaky_backward(gi, None, None, None, x, None, v, None, None, (alpha, 0), (None, 0), B, T, M, L, acc_decay=acc)
    assert ok is False
