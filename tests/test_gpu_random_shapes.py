"""Seeded random sweep over shapes, layouts, parameter modes and options, so that every kernel route
(TMA wide/narrow tiles, cp.async rings with 16/8/4-byte pieces, [N,T] 16-byte and 4-byte variants, leaky
warp scan) meets shapes nobody picked by hand.  Forward bit-exact against the checker, backward to 1e-5
against its float64 form.  Needs a GPU."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests._cases import lif_case, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-5

M_CHOICES = [1, 2, 3, 4, 6, 7, 8, 12, 30, 31, 33, 36, 64, 100, 127, 128, 130, 255, 258, 260, 511, 516, 640]


def _draw(seed):
    rng = np.random.default_rng(1000 + seed)
    B = int(rng.integers(1, 7))
    T = int(rng.choice([1, 2, 3, 5, 8, 17, 31, 32, 33, 47, 64, 65, 96, 100, 129]))
    M = int(rng.choice(M_CHOICES))
    if seed % 6 == 5:           # some problems wide enough for the 512-neuron TMA tiles
        B, M = int(rng.integers(150, 310)), int(rng.choice([516, 1024, 520]))
        T = int(rng.choice([3, 9, 14]))
    return rng, B, T, M


@pytest.mark.parametrize("seed", range(36))
def test_random_lif(seed):
    from sinabs_exodus_b200 import _lib
    from tests import _gpu
    rng, B, T, M = _draw(seed)
    N = B * M
    layout = int(rng.integers(0, 2))
    mode = int(rng.integers(0, 3))
    clamp = bool(rng.integers(0, 2))
    max_spikes = [None, 1, 3][int(rng.integers(0, 3))]
    cs = lif_case(seed, N, T, clamp=clamp)
    for k in ("alpha", "theta", "subtract", "theta_low"):
        if cs[k] is None:
            continue
        if mode == _lib.PARAM_SCALAR:
            cs[k] = np.full(N, cs[k][0], np.float32)
        elif mode == _lib.PARAM_PER_M:
            cs[k] = np.tile(cs[k][:M], B)
    s_ref, v_ref = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"],
                                   max_spikes)
    s, v, _, count = _gpu.lif_forward(cs, B, M, layout, mode, max_spikes)
    np.testing.assert_array_equal(v, v_ref)
    np.testing.assert_array_equal(s, s_ref)
    assert count == int(s_ref.sum())

    go = rng.standard_normal((N, T)).astype(np.float32)
    with_gv = bool(rng.integers(0, 2))
    gv = (0.3 * rng.standard_normal((N, T))).astype(np.float32) if with_gv else None
    kind, p0, p1, fn = [
        (_lib.SURR_SINGLE_EXPONENTIAL, 0.5, 1.0, lambda a, th: orc.surrogate_single_exponential(a, th, 0.5, 1.0)),
        (_lib.SURR_HEAVISIDE, 0.6, 0.0, lambda a, th: orc.surrogate_heaviside(a, th, 0.6)),
        (_lib.SURR_PERIODIC_EXPONENTIAL, 0.5, 1.0, lambda a, th: orc.surrogate_periodic_exponential(a, th, 0.5, 1.0)),
    ][int(rng.integers(0, 3))]
    surr = fn(v_ref, cs["theta"][:, None])
    nc = (v_ref > cs["theta_low"][:, None]).astype(np.float32) if clamp else np.ones_like(v_ref)
    g = (surr * go).astype(np.float32) + (gv if with_gv else 0)
    vpost = (v_ref - cs["subtract"][:, None] * s_ref).astype(np.float32)
    gi64, ga64 = orc.lif_backward_f64(g, surr, nc, cs["alpha"], cs["subtract"], vpost, cs["v_init"])
    gi, ga, g0, _ = _gpu.lif_backward(cs, v_ref, go, B, M, layout, mode=mode, gv=gv, kind=kind, p0=p0, p1=p1,
                                      max_spikes=max_spikes, want_alpha=True)
    assert rel_err(gi, gi64) < TOL
    assert rel_err(ga, ga64) < 2 * TOL
    assert rel_err(g0, cs["alpha"].astype(np.float64) * gi64[:, 0]) < TOL


@pytest.mark.parametrize("seed", range(24))
def test_random_lif_nt_row_classes(seed):
    """[N,T] layout on shapes the TMA-staged [N,T] kernels take (T % 4 == 0, T >= 64, N a multiple of the number of
    row classes) with B > 1 and all parameter modes: a CTA's rows are p rows apart there, so the (batch item, neuron)
    of a row is not the one of its neighbour."""
    from sinabs_exodus_b200 import _lib
    from tests import _gpu
    rng = np.random.default_rng(7000 + seed)
    B = int(rng.integers(1, 5))
    M = int(rng.choice([8, 16, 24, 40, 72, 136, 264]))
    T = int(rng.choice([64, 68, 72, 80, 96, 100, 132, 200, 260, 300]))
    N = B * M
    mode = int(rng.integers(0, 3))
    clamp = bool(rng.integers(0, 2))
    max_spikes = [None, 1, 3][int(rng.integers(0, 3))]
    cs = lif_case(900 + seed, N, T, clamp=clamp)
    for k in ("alpha", "theta", "subtract", "theta_low"):
        if cs[k] is None:
            continue
        if mode == _lib.PARAM_SCALAR:
            cs[k] = np.full(N, cs[k][0], np.float32)
        elif mode == _lib.PARAM_PER_M:
            cs[k] = np.tile(cs[k][:M], B)
    s_ref, v_ref = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"],
                                   max_spikes)
    s, v, v_post, count = _gpu.lif_forward(cs, B, M, _lib.LAYOUT_NT, mode, max_spikes)
    np.testing.assert_array_equal(v, v_ref)
    np.testing.assert_array_equal(s, s_ref)
    assert count == int(s_ref.sum())
    np.testing.assert_allclose(v_post, v_ref[:, -1].astype(np.float64) - cs["subtract"].astype(np.float64) * s_ref[:, -1],
                               rtol=1e-6, atol=1e-6)

    go = rng.standard_normal((N, T)).astype(np.float32)
    with_gv = bool(rng.integers(0, 2))
    gv = (0.3 * rng.standard_normal((N, T))).astype(np.float32) if with_gv else None
    kind, p0, p1, fn = [
        (_lib.SURR_SINGLE_EXPONENTIAL, 0.5, 1.0, lambda a, th: orc.surrogate_single_exponential(a, th, 0.5, 1.0)),
        (_lib.SURR_HEAVISIDE, 0.6, 0.0, lambda a, th: orc.surrogate_heaviside(a, th, 0.6)),
        (_lib.SURR_PERIODIC_EXPONENTIAL, 0.5, 1.0, lambda a, th: orc.surrogate_periodic_exponential(a, th, 0.5, 1.0)),
    ][int(rng.integers(0, 3))]
    surr = fn(v_ref, cs["theta"][:, None])
    nc = (v_ref > cs["theta_low"][:, None]).astype(np.float32) if clamp else np.ones_like(v_ref)
    g = (surr * go).astype(np.float32) + (gv if with_gv else 0)
    vpost = (v_ref - cs["subtract"][:, None] * s_ref).astype(np.float32)
    gi64, ga64 = orc.lif_backward_f64(g, surr, nc, cs["alpha"], cs["subtract"], vpost, cs["v_init"])
    gi, ga, g0, _ = _gpu.lif_backward(cs, v_ref, go, B, M, _lib.LAYOUT_NT, mode=mode, gv=gv, kind=kind, p0=p0, p1=p1,
                                      max_spikes=max_spikes, want_alpha=True)
    assert rel_err(gi, gi64) < TOL
    assert rel_err(ga, ga64) < 2 * TOL
    assert rel_err(g0, cs["alpha"].astype(np.float64) * gi64[:, 0]) < TOL


@pytest.mark.parametrize("seed", range(24))
def test_random_leaky(seed):
    from tests import _gpu
    rng, B, T, M = _draw(100 + seed)
    T = int(T * rng.choice([1, 1, 7]))          # some longer rows for the scans
    N = B * M
    layout = int(rng.integers(0, 2))
    mode = int(rng.integers(0, 3))
    x = rng.standard_normal((N, T)).astype(np.float32)
    go = rng.standard_normal((N, T)).astype(np.float32)
    base = rng.uniform(0.3, 1.0, N).astype(np.float32)
    alpha = base if mode == 2 else (np.tile(base[:M], B) if mode == 1 else np.full(N, base[0], np.float32))
    v0 = rng.standard_normal(N).astype(np.float32)
    out, v_last = _gpu.leaky_forward(x, v0, alpha, B, M, layout, mode)
    assert rel_err(out, orc.leaky_forward_f64(x, v0, alpha)) < TOL
    np.testing.assert_array_equal(v_last, out[:, -1])
    out_ref = orc.leaky_forward(x, v0, alpha)
    gi64, ag64 = orc.leaky_backward_f64(go, alpha, x, v0)
    gi, ga, g0, gs = _gpu.leaky_backward(go, alpha, B, M, layout, mode, out=out_ref, inp=x, v_init=v0,
                                         want_alpha=True, want_scale=True)
    assert rel_err(gi, gi64) < TOL
    assert rel_err(ga, ag64) < 2 * TOL
    assert rel_err(gs, (gi64 * x.astype(np.float64)).sum(1)) < 2 * TOL
