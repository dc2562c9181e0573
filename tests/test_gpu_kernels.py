"""Parity of the CUDA kernels (called through the C ABI) with the CPU checker.  Needs a GPU.

Forward results are compared bit for bit.  Gradients are compared with the
checker's float32 restatement of the reference loops and with its float64
ground truth under the 1e-5 criterion ``|a - ref| <= 1e-5 * max(|ref|, rms(ref))``.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from tests._cases import lif_case, near_threshold_rows, rel_err

pytestmark = pytest.mark.gpu

TOL = 1e-5

# the last two are wide enough (B * ceil(M/512) >= 296) for the 512-neuron TMA tiles
SHAPES = [(1, 1, 1), (2, 3, 5), (3, 33, 37), (2, 64, 128), (1, 100, 257), (4, 31, 32), (2, 130, 36), (5, 7, 4),
          (3, 50, 38), (4, 70, 6),            # M even but not a multiple of 4: two neurons per thread, 8-byte copies
          (300, 9, 516), (150, 21, 1024)]


def _tile_case(seed, B, T, M, mode, **kw):
    """Problem with N = B*M rows whose parameters are consistent with the parameter mode."""
    from sinabs_exodus_b200 import _lib
    N = B * M
    cs = lif_case(seed, N, T, **kw)
    for k in ("alpha", "theta", "subtract", "theta_low"):
        if cs[k] is None:
            continue
        if mode == _lib.PARAM_SCALAR:
            cs[k] = np.full(N, cs[k][0], np.float32)
        elif mode == _lib.PARAM_PER_M:
            cs[k] = np.tile(cs[k][:M], B)
    return cs


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("B,T,M", SHAPES)
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_lif_forward_bit_exact(layout, B, T, M, mode):
    from tests import _gpu
    for clamp, max_spikes in ((True, None), (False, 1), (True, 2)):
        cs = _tile_case(100 + B + T + M, B, T, M, mode, clamp=clamp)
        s_ref, v_ref = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"],
                                       cs["theta_low"], max_spikes)
        s, v, v_post, count = _gpu.lif_forward(cs, B, M, layout, mode, max_spikes)
        np.testing.assert_array_equal(v, v_ref)
        np.testing.assert_array_equal(s, s_ref)
        assert count == int(s_ref.sum())
        want_post = v_ref[:, -1].astype(np.float64) - cs["subtract"].astype(np.float64) * s_ref[:, -1]
        np.testing.assert_allclose(v_post, want_post, rtol=1e-6, atol=1e-6)


# T % 32 == 0: one row class; 16 / 8 / 4 mod 32: two / four / eight classes; N multiples of the class count that
# do not fill the last CTA, a single CTA, and many CTAs
NT_TMA_SHAPES = [(333, 96), (128, 64), (1000, 160), (31, 4000),
                 (334, 112), (130, 80), (1000, 72), (132, 104), (1000, 300), (136, 68), (8, 100), (2312, 300), (64, 1004)]


@pytest.mark.parametrize("N,T", NT_TMA_SHAPES)
@pytest.mark.parametrize("reset_mode", [0, 1])
def test_lif_forward_nt_tma_row_classes(N, T, reset_mode):
    """[N,T] layout with T % 4 == 0, the shapes the TMA-staged [N,T] forward takes: rows are grouped into classes that
    start at the same position inside a 128-byte line (one class when T % 32 == 0, up to eight otherwise), boxes of a
    class are placed on its lines, the first partial chunk of a class is stored by the threads, TMA stores clip at the
    ends of rows and of the tensor.  Bit-exact against the checker, for both reset modes."""
    from tests import _gpu
    from sinabs_exodus_b200 import _lib
    for clamp, max_spikes in ((True, None), (False, 1)):
        cs = _tile_case(7 + N + T, 1, T, N, 2, clamp=clamp)
        if reset_mode == 1:
            cs["subtract"] = (0.25 * cs["theta"]).astype(np.float32)
        s_ref, v_ref = orc.lif_forward_ext(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"],
                                           cs["theta_low"], max_spikes, reset_to_value=bool(reset_mode))
        s, v, v_post, count = _gpu.lif_forward(cs, 1, N, _lib.LAYOUT_NT, 2, max_spikes, reset_mode=reset_mode)
        np.testing.assert_array_equal(v, v_ref)
        np.testing.assert_array_equal(s, s_ref)
        assert count == int(s_ref.sum())
        assert s_ref.sum() > 0


@pytest.mark.parametrize("N,T", [(264, 300), (200, 96), (132, 104), (7, 300)])
@pytest.mark.parametrize("elem_offset", [4, 12, 32, 3])
def test_lif_forward_nt_tensors_inside_an_allocation(N, T, elem_offset):
    """The same with tensors that start 16, 48, 128 or 12 bytes into their allocations (a view into a larger buffer):
    every row then starts somewhere else inside its line; nothing outside the tensors may be written.  (7 rows: not a
    multiple of the eight classes; 12 bytes: not a 16-byte boundary -- both leave the TMA path.)"""
    from tests import _gpu
    from sinabs_exodus_b200 import _lib
    cs = _tile_case(11 + N + T + elem_offset, 1, T, N, 2, clamp=True)
    s_ref, v_ref = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"], None)
    s, v, v_post, count = _gpu.lif_forward(cs, 1, N, _lib.LAYOUT_NT, 2, None, elem_offset=elem_offset)
    np.testing.assert_array_equal(v, v_ref)
    np.testing.assert_array_equal(s, s_ref)
    assert count == int(s_ref.sum())


def test_lif_forward_defaults_and_strong_input():
    """subtract omitted (= threshold), no v_init, many spikes per step."""
    from tests import _gpu
    B, T, M = 2, 50, 64
    cs = lif_case(7, B * M, T, clamp=False, in_mean=2.0, in_std=1.5, subtract_given=False)
    s_ref, v_ref = orc.lif_forward(cs["inp"], np.zeros(B * M, np.float32), cs["alpha"], cs["theta"], cs["theta"])
    assert s_ref.max() >= 3
    cs2 = dict(cs, subtract=None, v_init=None)
    for layout in (0, 1):
        s, v, _, _ = _gpu.lif_forward(cs2, B, M, layout, 2)
        np.testing.assert_array_equal(v, v_ref)
        np.testing.assert_array_equal(s, s_ref)


def _surrogates():
    from sinabs_exodus_b200 import _lib
    return [
        ("generic", _lib.SURR_GENERIC, 0.0, 0.0, lambda v, th: orc.surrogate_single_exponential(v, th, 0.7, 1.3)),
        ("single_exp", _lib.SURR_SINGLE_EXPONENTIAL, 0.5, 1.0, lambda v, th: orc.surrogate_single_exponential(v, th, 0.5, 1.0)),
        ("heaviside", _lib.SURR_HEAVISIDE, 0.6, 0.0, lambda v, th: orc.surrogate_heaviside(v, th, 0.6)),
        ("periodic", _lib.SURR_PERIODIC_EXPONENTIAL, 0.5, 1.0, lambda v, th: orc.surrogate_periodic_exponential(v, th, 0.5, 1.0)),
    ]


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("B,T,M", [(2, 3, 5), (3, 33, 37), (2, 64, 128), (1, 100, 257), (4, 31, 32), (1, 1, 3), (300, 9, 516),
                                   (3, 50, 38), (2, 45, 6)])
@pytest.mark.parametrize("surr_idx", [0, 1, 2, 3])
def test_lif_backward_parity(layout, B, T, M, surr_idx):
    from tests import _gpu
    name, kind, p0, p1, fn = _surrogates()[surr_idx]
    N = B * M
    for clamp, max_spikes, with_gv in ((True, None, True), (False, 2, False)):
        cs = lif_case(300 + T + M, N, T, clamp=clamp)
        s, v = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"],
                               max_spikes)
        rng = np.random.default_rng(T * 7 + M)
        go = rng.standard_normal((N, T)).astype(np.float32)
        gv = (0.3 * rng.standard_normal((N, T))).astype(np.float32) if with_gv else None
        gi32, ga32, g032 = orc.integrate_and_fire_backward(
            go, gv if with_gv else np.zeros_like(go), v, s, cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"],
            cs["theta_low"], fn, True)
        surr = fn(v, cs["theta"][:, None])
        nc = (v > cs["theta_low"][:, None]).astype(np.float32) if clamp else np.ones_like(v)
        g = (surr * go).astype(np.float32) + (gv if with_gv else 0)
        vpost = (v - cs["subtract"][:, None] * s).astype(np.float32)
        gi64, ga64 = orc.lif_backward_f64(g, surr, nc, cs["alpha"], cs["subtract"], vpost, cs["v_init"])
        gi, ga, g0, _ = _gpu.lif_backward(cs, v, go, B, M, layout, gv=gv, surr=surr if kind == 0 else None,
                                          kind=kind, p0=p0, p1=p1, max_spikes=max_spikes, want_alpha=True)
        assert rel_err(gi, gi64) < TOL, name
        assert rel_err(gi, gi32) < 2 * TOL, name
        assert rel_err(ga, ga64) < TOL, name
        assert rel_err(g0, cs["alpha"].astype(np.float64) * gi64[:, 0]) < TOL, name
        # without alpha gradient the input gradient is the same
        gi_b, ga_b, _, _ = _gpu.lif_backward(cs, v, go, B, M, layout, gv=gv, surr=surr if kind == 0 else None,
                                             kind=kind, p0=p0, p1=p1, max_spikes=max_spikes, want_alpha=False)
        np.testing.assert_array_equal(gi_b, gi)
        assert ga_b is None


@pytest.mark.parametrize("N,T", [(264, 300), (200, 96), (136, 104), (1000, 72), (8, 100), (64, 1004), (128, 64)])
@pytest.mark.parametrize("surr_idx", [0, 1, 2, 3])
def test_lif_backward_nt_tma_row_classes(N, T, surr_idx):
    """[N,T] layout with T % 4 == 0, the shapes the TMA-staged [N,T] backward takes (one, two, four or eight row
    classes; rows that do not fill the last CTA of a class; a first chunk that the warps store themselves): input,
    alpha and initial-state gradients against the float64 form and the float32 restatement of the reference loops,
    with and without a gradient on v_mem, with and without the alpha gradient."""
    from tests import _gpu
    name, kind, p0, p1, fn = _surrogates()[surr_idx]
    for clamp, max_spikes, with_gv in ((True, None, True), (False, 2, False)):
        cs = lif_case(500 + T + N, N, T, clamp=clamp)
        s, v = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"],
                               max_spikes)
        rng = np.random.default_rng(T * 5 + N)
        go = rng.standard_normal((N, T)).astype(np.float32)
        gv = (0.3 * rng.standard_normal((N, T))).astype(np.float32) if with_gv else None
        gi32, ga32, g032 = orc.integrate_and_fire_backward(
            go, gv if with_gv else np.zeros_like(go), v, s, cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"],
            cs["theta_low"], fn, True)
        surr = fn(v, cs["theta"][:, None])
        nc = (v > cs["theta_low"][:, None]).astype(np.float32) if clamp else np.ones_like(v)
        g = (surr * go).astype(np.float32) + (gv if with_gv else 0)
        vpost = (v - cs["subtract"][:, None] * s).astype(np.float32)
        gi64, ga64 = orc.lif_backward_f64(g, surr, nc, cs["alpha"], cs["subtract"], vpost, cs["v_init"])
        gi, ga, g0, _ = _gpu.lif_backward(cs, v, go, 1, N, 0, gv=gv, surr=surr if kind == 0 else None,
                                          kind=kind, p0=p0, p1=p1, max_spikes=max_spikes, want_alpha=True)
        assert np.isfinite(gi).all()
        assert rel_err(gi, gi64) < TOL, name
        assert rel_err(gi, gi32) < 2 * TOL, name
        assert rel_err(ga, ga64) < TOL, name
        assert rel_err(g0, cs["alpha"].astype(np.float64) * gi64[:, 0]) < TOL, name
        gi_b, ga_b, _, _ = _gpu.lif_backward(cs, v, go, 1, N, 0, gv=gv, surr=surr if kind == 0 else None,
                                             kind=kind, p0=p0, p1=p1, max_spikes=max_spikes, want_alpha=False)
        np.testing.assert_array_equal(gi_b, gi)
        assert ga_b is None


@pytest.mark.parametrize("N,T", [(264, 300), (136, 104), (128, 64)])
def test_lif_backward_nt_tma_scale_and_state_gradient(N, T):
    """The same kernels with a fused input scale (its gradient from the input tensor and rebuilt from v_mem) and a
    gradient arriving on the post-reset last state."""
    from tests import _gpu
    from sinabs_exodus_b200 import _lib
    cs = lif_case(79 + N, N, T, clamp=True)
    cs["alpha"] = np.minimum(cs["alpha"], np.float32(0.97))
    scale = (1.0 - cs["alpha"]).astype(np.float32)
    scaled = dict(cs, inp=(scale[:, None] * cs["inp"]).astype(np.float32))
    s_ref, v_ref = orc.lif_forward(scaled["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"])
    rng = np.random.default_rng(9 + T)
    go = rng.standard_normal((N, T)).astype(np.float32)
    G = rng.standard_normal(N).astype(np.float32)
    fn = lambda vv, th: orc.surrogate_single_exponential(vv, th)
    go2 = go.copy(); go2[:, -1] -= cs["subtract"] * G
    gv2 = np.zeros_like(go); gv2[:, -1] += G
    surr = fn(v_ref, cs["theta"][:, None])
    nc = (v_ref > cs["theta_low"][:, None]).astype(np.float32)
    g = (surr * go2).astype(np.float32) + gv2
    R64, _ = orc.lif_backward_f64(g, surr, nc, cs["alpha"], cs["subtract"])
    for from_state in (False, True):
        gi, _, g0, gs = _gpu.lif_backward(cs, v_ref, go, 1, N, 0, g_last=G, kind=_lib.SURR_SINGLE_EXPONENTIAL,
                                          p0=0.5, p1=1.0, in_scale=scale, want_scale=True, scale_from_state=from_state)
        assert rel_err(gi, scale[:, None].astype(np.float64) * R64) < TOL
        assert rel_err(gs, (R64 * cs["inp"].astype(np.float64)).sum(1)) < TOL
        assert rel_err(g0, cs["alpha"].astype(np.float64) * R64[:, 0]) < TOL


def test_first_step_clip_term_gpu():
    """Rows that start clipped with a non-zero initial state (reference cuda/lif_kernels.h:219-238)."""
    from tests import _gpu
    from sinabs_exodus_b200 import _lib
    N, T = 8, 12
    cs = lif_case(5, N, T, clamp=True)
    cs["inp"][:, 0] = -6.0
    cs["v_init"] = np.linspace(-0.4, 0.9, N).astype(np.float32)
    s, v = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"])
    assert (v[:, 0] == cs["theta_low"]).all()
    go = np.random.default_rng(1).standard_normal((N, T)).astype(np.float32)
    fn = lambda vv, th: orc.surrogate_single_exponential(vv, th)
    _, ga32, _ = orc.integrate_and_fire_backward(go, np.zeros_like(go), v, s, cs["v_init"], cs["alpha"],
                                                 cs["subtract"], cs["theta"], cs["theta_low"], fn, True)
    for layout, (B, M) in ((0, (1, N)), (1, (2, 4))):
        _, ga, _, _ = _gpu.lif_backward(cs, v, go, B, M, layout, kind=_lib.SURR_SINGLE_EXPONENTIAL, p0=0.5, p1=1.0,
                                        want_alpha=True)
        assert rel_err(ga, ga32) < TOL


@pytest.mark.parametrize("layout", [0, 1])
def test_in_scale_and_state_gradient(layout):
    """Fused input scale (+ its gradient) and a gradient arriving on the post-reset last state."""
    from tests import _gpu
    from sinabs_exodus_b200 import _lib
    B, T, M = 3, 40, 20
    N = B * M
    cs = lif_case(77, N, T, clamp=True)
    cs["alpha"] = np.minimum(cs["alpha"], np.float32(0.97))
    scale = (1.0 - cs["alpha"]).astype(np.float32)
    scaled = dict(cs, inp=(scale[:, None] * cs["inp"]).astype(np.float32))
    s_ref, v_ref = orc.lif_forward(scaled["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"])
    s, v, _, _ = _gpu.lif_forward(cs, B, M, layout, 2, in_scale=scale)
    np.testing.assert_array_equal(v, v_ref)
    np.testing.assert_array_equal(s, s_ref)

    rng = np.random.default_rng(9)
    go = rng.standard_normal((N, T)).astype(np.float32)
    G = rng.standard_normal(N).astype(np.float32)
    fn = lambda vv, th: orc.surrogate_single_exponential(vv, th)
    # the state gradient enters through the last step: go -= c*G, gv += G
    go2 = go.copy(); go2[:, -1] -= cs["subtract"] * G
    gv2 = np.zeros_like(go); gv2[:, -1] += G
    surr = fn(v_ref, cs["theta"][:, None])
    nc = (v_ref > cs["theta_low"][:, None]).astype(np.float32)
    g = (surr * go2).astype(np.float32) + gv2
    R64, _ = orc.lif_backward_f64(g, surr, nc, cs["alpha"], cs["subtract"])
    gi, _, g0, gs = _gpu.lif_backward(cs, v_ref, go, B, M, layout, g_last=G, kind=_lib.SURR_SINGLE_EXPONENTIAL,
                                      p0=0.5, p1=1.0, in_scale=scale, want_scale=True)
    assert rel_err(gi, scale[:, None].astype(np.float64) * R64) < TOL
    assert rel_err(gs, (R64 * cs["inp"].astype(np.float64)).sum(1)) < TOL
    assert rel_err(g0, cs["alpha"].astype(np.float64) * R64[:, 0]) < TOL
    # the same scale gradient rebuilt from v_mem alone (no input tensor passed), with and without alpha gradient
    for want_alpha in (False, True):
        gi2, _, _, gs2 = _gpu.lif_backward(cs, v_ref, go, B, M, layout, g_last=G, kind=_lib.SURR_SINGLE_EXPONENTIAL,
                                           p0=0.5, p1=1.0, in_scale=scale, want_scale=True, scale_from_state=True,
                                           want_alpha=want_alpha)
        np.testing.assert_array_equal(gi2, gi)
        assert rel_err(gs2, (R64 * cs["inp"].astype(np.float64)).sum(1)) < TOL


@pytest.mark.parametrize("B,T,M", [(3, 40, 20), (300, 9, 516), (3, 40, 21), (2, 37, 22)])
def test_backward_all_five_streams(B, T, M):
    """Time-major backward with every optional tensor streamed at once: grad_v_mem, a caller-computed
    surrogate, and the forward input for the scale gradient (narrow and wide TMA tiles)."""
    from tests import _gpu
    from sinabs_exodus_b200 import _lib
    N = B * M
    cs = lif_case(55, N, T, clamp=True)
    cs["alpha"] = np.minimum(cs["alpha"], np.float32(0.97))
    scale = (1.0 - cs["alpha"]).astype(np.float32)
    scaled = (scale[:, None] * cs["inp"]).astype(np.float32)
    s, v = orc.lif_forward(scaled, cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"])
    rng = np.random.default_rng(3)
    go = rng.standard_normal((N, T)).astype(np.float32)
    gv = (0.3 * rng.standard_normal((N, T))).astype(np.float32)
    surr = orc.surrogate_single_exponential(v, cs["theta"][:, None], 0.7, 1.3)
    nc = (v > cs["theta_low"][:, None]).astype(np.float32)
    g = (surr * go).astype(np.float32) + gv
    vpost = (v - cs["subtract"][:, None] * s).astype(np.float32)
    R64, ag64 = orc.lif_backward_f64(g, surr, nc, cs["alpha"], cs["subtract"], vpost, cs["v_init"])
    gi, ga, g0, gs = _gpu.lif_backward(cs, v, go, B, M, 1, gv=gv, surr=surr, kind=_lib.SURR_GENERIC,
                                       in_scale=scale, want_scale=True, want_alpha=True)
    assert rel_err(gi, scale[:, None].astype(np.float64) * R64) < TOL
    assert rel_err(ga, ag64) < TOL
    assert rel_err(gs, (R64 * cs["inp"].astype(np.float64)).sum(1)) < TOL


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("B,T,M", [(2, 30, 9), (2, 68, 8)])      # the second: TMA-staged kernels in both layouts
def test_reset_to_value_vs_bptt(layout, B, T, M):
    """Reset-to-value has no reference kernel; the checker is back-propagation through the time-stepped loop."""
    import torch
    from oracle.torch_loop import lif_loop
    from sinabs_exodus_b200 import _lib
    from sinabs_exodus_b200.compat.activation import SingleExponential
    from tests import _gpu
    N = B * M
    cs = lif_case(13, N, T, clamp=True)
    cs["subtract"] = np.full(N, 0.1, np.float32)      # the reset value
    cs["v_init"] = np.abs(cs["v_init"]) * 0.5
    x = torch.tensor(cs["inp"]).view(B, M, T).permute(0, 2, 1).contiguous().requires_grad_(True)
    alpha = torch.tensor(cs["alpha"]).view(B, M).requires_grad_(True)
    v0 = torch.tensor(cs["v_init"]).view(B, M).requires_grad_(True)
    res = lif_loop(x, alpha, v0, torch.tensor(cs["theta"]).view(B, M), None, torch.tensor(cs["theta_low"]).view(B, M),
                   SingleExponential(), 1, reset_value=0.1)
    rng = np.random.default_rng(4)
    go = rng.standard_normal((N, T)).astype(np.float32)
    G = rng.standard_normal(N).astype(np.float32)
    loss = (res["spikes"] * torch.tensor(go).view(B, M, T).permute(0, 2, 1)).sum() + (res["v_last"] * torch.tensor(G).view(B, M)).sum()
    loss.backward()
    s, v, v_post, _ = _gpu.lif_forward(cs, B, M, layout, 2, max_spikes=1, reset_mode=_lib.RESET_TO_VALUE)
    s_ref = res["spikes"].detach().permute(0, 2, 1).reshape(N, T).numpy()
    v_ref = res["v_mem_pre"].detach().permute(0, 2, 1).reshape(N, T).numpy()
    safe = ~near_threshold_rows(v_ref, cs["theta"])
    np.testing.assert_array_equal(s[safe], s_ref[safe])
    assert rel_err(v[safe], v_ref[safe]) < TOL
    assert rel_err(v_post[safe], res["v_last"].detach().reshape(N).numpy()[safe]) < TOL
    gi, ga, g0, _ = _gpu.lif_backward(cs, v, go, B, M, layout, g_last=G, kind=_lib.SURR_SINGLE_EXPONENTIAL, p0=0.5,
                                      p1=1.0, max_spikes=1, reset_mode=_lib.RESET_TO_VALUE, want_alpha=True)
    assert rel_err(gi[safe], x.grad.permute(0, 2, 1).reshape(N, T).numpy()[safe]) < 5 * TOL
    assert rel_err(ga[safe], alpha.grad.reshape(N).numpy()[safe]) < 5 * TOL
    assert rel_err(g0[safe], v0.grad.reshape(N).numpy()[safe]) < 5 * TOL


LEAKY_SHAPES = [(1, 1, 1), (2, 3, 5), (3, 33, 37), (2, 64, 128), (1, 300, 7), (2, 129, 4), (1, 1000, 3), (4, 128, 8),
                (3, 60, 6), (2, 41, 38),             # M even, not a multiple of 4: two neurons per thread
                (300, 11, 516), (140, 7, 644)]   # last two: 512-neuron and 128-neuron TMA tiles


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("B,T,M", LEAKY_SHAPES)
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_leaky_parity(layout, B, T, M, mode):
    from tests import _gpu
    N = B * M
    rng = np.random.default_rng(B * 1000 + T * 10 + M)
    x = rng.standard_normal((N, T)).astype(np.float32)
    go = rng.standard_normal((N, T)).astype(np.float32)
    base = rng.uniform(0.3, 1.0, N).astype(np.float32)
    alpha = base if mode == 2 else (np.tile(base[:M], B) if mode == 1 else np.full(N, base[0], np.float32))
    v0 = rng.standard_normal(N).astype(np.float32)
    G = rng.standard_normal(N).astype(np.float32)
    out_ref = orc.leaky_forward(x, v0, alpha)
    out, v_last = _gpu.leaky_forward(x, v0, alpha, B, M, layout, mode)
    if layout == 1:
        np.testing.assert_array_equal(out, out_ref)          # sequential sweep: same roundings
    assert rel_err(out, orc.leaky_forward_f64(x, v0, alpha)) < TOL
    np.testing.assert_array_equal(v_last, out[:, -1])
    go2 = go.copy(); go2[:, -1] += G
    gi64, ag64 = orc.leaky_backward_f64(go2, alpha, x, v0)
    gi, ga, g0, gs = _gpu.leaky_backward(go, alpha, B, M, layout, mode, out=out_ref, inp=x, v_init=v0, g_last=G,
                                         want_alpha=True, want_scale=True)
    assert rel_err(gi, gi64) < TOL
    assert rel_err(ga, ag64) < 2 * TOL
    assert rel_err(g0, alpha.astype(np.float64) * gi64[:, 0]) < TOL
    assert rel_err(gs, (gi64 * x.astype(np.float64)).sum(1)) < 2 * TOL
    gi_b, ga_b, _, _ = _gpu.leaky_backward(go, alpha, B, M, layout, mode, g_last=G)
    np.testing.assert_array_equal(gi_b, gi)
    if layout == 1:
        np.testing.assert_array_equal(gi, orc.leaky_backward(go2, alpha))


def test_leaky_in_scale():
    from tests import _gpu
    B, T, M = 2, 50, 16
    N = B * M
    rng = np.random.default_rng(8)
    x = rng.standard_normal((N, T)).astype(np.float32)
    alpha = rng.uniform(0.5, 1.0, N).astype(np.float32)
    v0 = rng.standard_normal(N).astype(np.float32)
    xs = (alpha[:, None] * x).astype(np.float32)
    ref = orc.leaky_forward(xs, v0, alpha)
    for layout in (0, 1):
        out, _ = _gpu.leaky_forward(x, v0, alpha, B, M, layout, 2, in_scale=alpha)
        assert rel_err(out, ref) < TOL
        go = rng.standard_normal((N, T)).astype(np.float32)
        gi64, _ = orc.leaky_backward_f64(go, alpha)
        gi, _, _, gs = _gpu.leaky_backward(go, alpha, B, M, layout, 2, inp=x, in_scale=alpha, want_scale=True)
        assert rel_err(gi, alpha[:, None] * gi64) < TOL
        assert rel_err(gs, (gi64 * x).sum(1)) < 2 * TOL


@pytest.mark.parametrize("B,T,M", [(1, 4000, 128), (2, 1000, 36), (1, 5003, 4), (3, 777, 260), (1, 20000, 8)])
@pytest.mark.parametrize("mode", [0, 2])
def test_leaky_time_parallel_scan(B, T, M, mode):
    """Long sequences with few neurons: the time axis is split across CTAs (needs scratch memory)."""
    from sinabs_exodus_b200 import _lib
    from tests import _gpu
    N = B * M
    assert _lib.leaky_scan_workspace_bytes(B, T, M) > 0
    rng = np.random.default_rng(T + M)
    x = rng.standard_normal((N, T)).astype(np.float32)
    go = rng.standard_normal((N, T)).astype(np.float32)
    base = rng.uniform(0.8, 1.0, N).astype(np.float32)
    alpha = base if mode == 2 else np.full(N, base[0], np.float32)
    scale = (1.0 - alpha).astype(np.float32)
    v0 = rng.standard_normal(N).astype(np.float32)
    G = rng.standard_normal(N).astype(np.float32)
    xs = (scale[:, None] * x).astype(np.float32)
    out, v_last = _gpu.leaky_forward_scan(x, v0, alpha, B, M, mode, in_scale=scale)
    ref = orc.leaky_forward_f64(xs, v0, alpha)
    assert rel_err(out, ref) < TOL
    np.testing.assert_array_equal(v_last, out[:, -1])
    # same answer (to rounding) as the sequential entry point
    out_seq, _ = _gpu.leaky_forward(x, v0, alpha, B, M, 1, mode, in_scale=scale)
    assert rel_err(out, out_seq) < TOL
    go2 = go.copy(); go2[:, -1] += G
    gi64, ag64 = orc.leaky_backward_f64(go2, alpha, xs, v0)
    out32 = orc.leaky_forward(xs, v0, alpha)
    for _ in range(2):      # twice: the scratch memory is reused
        gi, ga, g0, gs = _gpu.leaky_backward_scan(go, alpha, B, M, mode, out=out32, inp=x, v_init=v0, g_last=G,
                                                  in_scale=scale, want_alpha=True, want_scale=True)
        assert rel_err(gi, scale[:, None] * gi64) < TOL
        assert rel_err(ga, ag64) < 2 * TOL
        assert rel_err(g0, alpha.astype(np.float64) * gi64[:, 0]) < TOL
        assert rel_err(gs, (gi64 * x.astype(np.float64)).sum(1)) < 2 * TOL
    gi_b, ga_b, _, _ = _gpu.leaky_backward_scan(go, alpha, B, M, mode, g_last=G, in_scale=scale)
    np.testing.assert_array_equal(gi_b, gi)


def test_leaky_scan_not_applicable():
    from sinabs_exodus_b200 import _lib
    assert _lib.leaky_scan_workspace_bytes(4, 100, 128) == 0        # too short to split
    assert _lib.leaky_scan_workspace_bytes(1, 4000, 130) == 0       # M % 4 != 0: no TMA
    assert _lib.leaky_scan_workspace_bytes(64, 4000, 8192) == 0     # enough tiles already


def test_golden_vectors_gpu():
    """The CUDA path against the committed outputs of the reference's kernels."""
    import glob, os
    from tests import _gpu
    files = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
    if not files:
        pytest.skip("no golden vectors committed yet")
    for path in files:
        g = dict(np.load(path))
        N = g["inp"].shape[0]
        if str(g["kind"]) == "lif":
            cs = dict(inp=g["inp"], v_init=g["v_init"], alpha=g["alpha"], subtract=g["subtract"], theta=g["theta"],
                      theta_low=g["theta_low"] if g["apply_theta_low"] else None)
            ms = None if int(g["max_spikes"]) < 0 else int(g["max_spikes"])
            for layout in (0, 1):
                s, v, _, _ = _gpu.lif_forward(cs, 1, N, layout, 2, ms)
                np.testing.assert_array_equal(v, g["ref_v_mem"])
                np.testing.assert_array_equal(s, g["ref_spikes"])
                # the stored g already is surr*go + gv: feed it as go' = 0, gv' = g
                gi, ga, _, _ = _gpu.lif_backward(cs, g["ref_v_mem"], np.zeros_like(g["g"]), 1, N, layout, gv=g["g"],
                                                 surr=g["surr"], max_spikes=ms, want_alpha=True)
                assert rel_err(gi, g["ref_grad_input"]) < TOL
                assert rel_err(ga, g["ref_grad_alpha"]) < TOL
        else:
            for layout in (0, 1):
                out, _ = _gpu.leaky_forward(g["inp"], g["v_init"], g["alpha"], 1, N, layout, 2)
                assert rel_err(out, g["ref_out"]) < TOL
                gi, ga, _, _ = _gpu.leaky_backward(g["go"], g["alpha"], 1, N, layout, 2, out=g["ref_out"],
                                                   v_init=g["v_init"], want_alpha=True)
                assert rel_err(gi, g["ref_grad_input"]) < TOL
                assert rel_err(ga, g["ref_grad_alpha"]) < TOL


def test_device_status_clean():
    """After all the launches above no bounded device-side wait has run out."""
    from sinabs_exodus_b200 import _lib
    _lib.device_status()


@pytest.mark.parametrize("B,T,M", [(3, 33, 37), (2, 40, 38), (2, 64, 128), (300, 9, 516)])
@pytest.mark.parametrize("reset_mode", [0, 1])
def test_forward_record_of_post_reset_potential(B, T, M, reset_mode):
    """exb_lif_forward_record: the extra output equals v_mem - subtract * spikes (two roundings, as PyTorch
    forms it) or the reset value where a spike occurred; spikes and v_mem are those of exb_lif_forward.
    Shapes cover the cp.async rings (4- and 8-byte pieces) and both TMA tile widths."""
    import torch
    from sinabs_exodus_b200 import _lib
    from tests import _gpu
    cs = _tile_case(40 + M, B, T, M, _lib.PARAM_PER_N, clamp=True)
    N = B * M
    x = _gpu.to_dev(cs["inp"], B, M, _lib.LAYOUT_BTM)
    spikes, v_mem, rec = (torch.full_like(x, float("nan")) for _ in range(3))
    par = lambda k: _gpu.param(cs[k], _lib.PARAM_PER_N, B, M)
    _lib.lif_forward(spikes, v_mem, x, _gpu.vec(cs["v_init"]), (None, 0), par("alpha"), par("subtract"), par("theta"),
                     par("theta_low"), None, reset_mode, None, None, B, T, M, _lib.LAYOUT_BTM, v_post=rec)
    s2, v2 = torch.full_like(x, float("nan")), torch.full_like(x, float("nan"))
    _lib.lif_forward(s2, v2, x, _gpu.vec(cs["v_init"]), (None, 0), par("alpha"), par("subtract"), par("theta"),
                     par("theta_low"), None, reset_mode, None, None, B, T, M, _lib.LAYOUT_BTM)
    torch.cuda.synchronize()
    assert torch.equal(spikes, s2) and torch.equal(v_mem, v2)
    c = torch.as_tensor(cs["subtract"], device=x.device).view(B, 1, M)
    want = v_mem - c * spikes if reset_mode == _lib.RESET_SUBTRACT else torch.where(spikes > 0, c.expand_as(v_mem), v_mem)
    assert torch.equal(rec, want)
    with pytest.raises(_lib.ExodusLibraryError):      # the [N,T] kernels do not write it
        _lib.lif_forward(spikes, v_mem, x, _gpu.vec(cs["v_init"]), (None, 0), par("alpha"), par("subtract"),
                         par("theta"), par("theta_low"), None, reset_mode, None, None, 1, T, N, _lib.LAYOUT_NT, v_post=rec)
