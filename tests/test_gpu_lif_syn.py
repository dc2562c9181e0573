"""exb_lif_syn_forward / exb_lif_syn_backward through the C ABI against the CPU checker.  Needs a GPU.

Forward: the synaptic current must equal the checker's leaky integrator on the pre-scaled input bit for bit, and
spikes / membrane potential the checker's spike scan on that current (the two-kernel chain of the reference layer,
layers/lif.py:185-258, gives exactly these roundings).  Backward: input gradient, both initial-state gradients and
the four per-instance parameter gradients against the float64 adjoint of the same chain, 1e-5, for both reset
modes, every surrogate, narrow and wide tiles, every parameter mode, with and without the optional gradient inputs.
"""
import zlib

import numpy as np
import pytest

from oracle import oracle as orc
from sinabs_exodus_b200 import _lib
from tests import _gpu
from tests._cases import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-5

SURROGATES = {
    "generic": (_lib.SURR_GENERIC, 0.0, 0.0),
    "single_exponential": (_lib.SURR_SINGLE_EXPONENTIAL, 0.5, 1.0),
    "heaviside": (_lib.SURR_HEAVISIDE, 0.7, 0.0),
    "periodic_exponential": (_lib.SURR_PERIODIC_EXPONENTIAL, 0.5, 1.0),
}

# (B, T, M, parameter mode): narrow tiles (one neuron per thread) while B*ceil(M/512) < 296, wide tiles beyond
SHAPES = {
    "narrow_per_n": (3, 37, 64, _lib.PARAM_PER_N),
    "narrow_per_m_ragged_tile": (5, 23, 132, _lib.PARAM_PER_M),
    "narrow_scalar_long": (2, 301, 8, _lib.PARAM_SCALAR),
    "wide_scalar": (37, 9, 4096, _lib.PARAM_SCALAR),
    "wide_per_m": (37, 11, 4096, _lib.PARAM_PER_M),
    "wide_per_n_ragged_tile": (75, 7, 2052, _lib.PARAM_PER_N),
}


def synaptic_case(seed, B, T, M, mode, clamp, reset_to_value):
    """Random two-stage problem in the [N,T] layout whose per-neuron vectors are consistent with `mode`."""
    rng = np.random.default_rng(seed)
    N = B * M

    def per(lo, hi):
        if mode == _lib.PARAM_SCALAR:
            return np.full(N, rng.uniform(lo, hi), np.float32)
        if mode == _lib.PARAM_PER_M:
            return np.tile(rng.uniform(lo, hi, M).astype(np.float32), B)
        return rng.uniform(lo, hi, N).astype(np.float32)

    cs = dict(inp=(0.3 + 1.2 * rng.standard_normal((N, T))).astype(np.float32),
              a_syn=per(0.5, 0.95), s_syn=per(0.5, 1.0), a_mem=per(0.5, 0.98), s_mem=per(0.2, 0.6),
              theta=per(0.4, 1.1), theta_low=(-per(0.2, 0.8)) if clamp else None,
              v_init=rng.uniform(-0.4, 0.4, N).astype(np.float32), i_init=rng.uniform(-0.4, 0.4, N).astype(np.float32))
    cs["subtract"] = per(0.05, 0.3) if reset_to_value else (cs["theta"] * per(0.5, 1.0)).astype(np.float32)
    return cs


def reference_forward(cs, max_spikes, reset_to_value):
    pre = (cs["s_syn"][:, None] * cs["inp"]).astype(np.float32)
    i_syn = orc.leaky_forward(pre, cs["i_init"], cs["a_syn"])
    s, v = orc.lif_forward_ext(i_syn, cs["v_init"], cs["a_mem"], cs["subtract"], cs["theta"], cs["theta_low"],
                               max_spikes, in_scale=cs["s_mem"], reset_to_value=reset_to_value)
    return s, v, i_syn


def surrogate_values(name, v, theta):
    if name == "generic":
        return 0.6 / (1.0 + 4.0 * (np.asarray(v, np.float64) - theta) ** 2)
    _, p0, p1 = SURROGATES[name]
    return orc.surrogate_f64(name, v, theta, p0, p1 if p1 else 1.0)


@pytest.mark.parametrize("reset_to_value", [False, True], ids=["subtract", "to_value"])
@pytest.mark.parametrize("shape", sorted(SHAPES))
@pytest.mark.parametrize("max_spikes", [None, 1])
def test_lif_syn_forward(shape, reset_to_value, max_spikes):
    B, T, M, mode = SHAPES[shape]
    cs = synaptic_case(zlib.crc32(shape.encode()) % 1000, B, T, M, mode, clamp=True, reset_to_value=reset_to_value)
    reset = _lib.RESET_TO_VALUE if reset_to_value else _lib.RESET_SUBTRACT
    got = _gpu.lif_syn_forward(cs["inp"], cs["v_init"], cs["i_init"], cs["a_syn"], cs["s_syn"], cs["s_mem"], cs["a_mem"],
                               cs["subtract"], cs["theta"], cs["theta_low"], B, M, mode, max_spikes, reset)
    assert got is not None
    s, v, i_syn, v_post, i_last, count = got
    s_ref, v_ref, i_ref = reference_forward(cs, max_spikes, reset_to_value)
    np.testing.assert_array_equal(i_syn, i_ref)
    np.testing.assert_array_equal(v, v_ref)
    np.testing.assert_array_equal(s, s_ref)
    np.testing.assert_array_equal(i_last, i_ref[:, -1])
    # the state after the last reset: one fused multiply-add in the kernel, i.e. the exact difference rounded once
    post = np.where(s_ref[:, -1] > 0, cs["subtract"], v_ref[:, -1]) if reset_to_value else \
        (v_ref[:, -1].astype(np.float64) - cs["subtract"].astype(np.float64) * s_ref[:, -1]).astype(np.float32)
    np.testing.assert_array_equal(v_post, post)
    assert count == int(s_ref.sum(dtype=np.float64))
    assert s_ref.sum() > 0 and (max_spikes == 1 or (s_ref > 1).any())


@pytest.mark.parametrize("reset_to_value", [False, True], ids=["subtract", "to_value"])
@pytest.mark.parametrize("surrogate", sorted(SURROGATES))
@pytest.mark.parametrize("shape", sorted(SHAPES))
@pytest.mark.parametrize("optional", ["plain", "all_gradients"])
def test_lif_syn_backward(shape, surrogate, reset_to_value, optional):
    B, T, M, mode = SHAPES[shape]
    everything = optional == "all_gradients"
    max_spikes = 1 if (reset_to_value and not everything) else None
    cs = synaptic_case(zlib.crc32((shape + surrogate).encode()) % 1000, B, T, M, mode, clamp=everything, reset_to_value=reset_to_value)
    reset = _lib.RESET_TO_VALUE if reset_to_value else _lib.RESET_SUBTRACT
    s, v, i_syn = reference_forward(cs, max_spikes, reset_to_value)
    N = B * M
    rng = np.random.default_rng(7)
    go = rng.standard_normal((N, T)).astype(np.float32)
    extra = dict(gv=None, g_vlast=None, g_isyn=None, g_ilast=None)
    if everything:
        extra = dict(gv=rng.standard_normal((N, T)).astype(np.float32), g_vlast=rng.standard_normal(N).astype(np.float32),
                     g_isyn=rng.standard_normal((N, T)).astype(np.float32), g_ilast=rng.standard_normal(N).astype(np.float32))
    kind, p0, p1 = SURROGATES[surrogate]
    surr64 = surrogate_values(surrogate, v, cs["theta"][:, None])
    surr32 = surr64.astype(np.float32) if surrogate == "generic" else None
    got = _gpu.lif_syn_backward(go, v, i_syn, cs["v_init"], cs["i_init"], cs["a_syn"], cs["s_syn"], cs["s_mem"], cs["a_mem"],
                                cs["subtract"], cs["theta"], cs["theta_low"], B, M, mode, max_spikes, reset, kind, p0, p1,
                                surr=surr32, want_params=True, want_init=True, **extra)
    ref = orc.lif_syn_backward_f64(go, v, s, i_syn, cs["inp"], surr32 if surrogate == "generic" else surr64,
                                   cs["v_init"], cs["i_init"], cs["a_syn"], cs["s_syn"], cs["s_mem"], cs["a_mem"],
                                   cs["subtract"], cs["theta_low"], reset_to_value, grad_v_mem=extra["gv"],
                                   grad_v_last=extra["g_vlast"], grad_i_syn=extra["g_isyn"], grad_i_last=extra["g_ilast"])
    errs = {k: rel_err(got[k], ref[k]) for k in ref}
    assert max(errs.values()) < TOL, errs
    # without the parameter gradients (i_syn is then not streamed) the input gradient is the same
    lean = _gpu.lif_syn_backward(go, v, i_syn, cs["v_init"], cs["i_init"], cs["a_syn"], cs["s_syn"], cs["s_mem"], cs["a_mem"],
                                 cs["subtract"], cs["theta"], cs["theta_low"], B, M, mode, max_spikes, reset, kind, p0, p1,
                                 surr=surr32, want_params=False, want_init=False, **extra)
    np.testing.assert_array_equal(lean["grad_input"], got["grad_input"])
    assert lean["grad_alpha_mem"] is None and lean["grad_v_init"] is None
