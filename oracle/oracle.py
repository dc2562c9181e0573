"""numpy front-end of the CPU checker (test infrastructure, never shipped).

Wraps ``oracle/_build/liboracle.so`` (built by ``oracle/build.py`` from
``exodus_oracle.c``) and restates, in numpy, the tensor glue the reference's
autograd Functions put around their kernels:

* ``IntegrateAndFire.backward``  -- sinabs/exodus/spike.py:229-291
* ``LeakyIntegrator.backward``   -- sinabs/exodus/leaky.py:53-76

Only ``tests/``, the smoke check and the benchmark's CPU-baseline leg import
this module.  Parity status: pinned by ``tests/golden`` (outputs of the
reference's kernels on a B200); the surrogate-gradient formulas are this
project's own definitions (the reference takes them from a separate package
that is not part of its source tree) and are therefore unpinned.
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBS = {}

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)


def _load(fma: bool = True) -> ctypes.CDLL:
    key = "fma" if fma else "nofma"
    if key not in _LIBS:
        name = "liboracle.so" if fma else "liboracle_nofma.so"
        path = os.path.join(_HERE, "_build", name)
        if not os.path.exists(path):
            from . import build as _b  # type: ignore
            _b.build_oracle()
        _LIBS[key] = ctypes.CDLL(path)
    return _LIBS[key]


def _p(a: Optional[np.ndarray], typ=_f32p):
    if a is None:
        return ctypes.cast(None, typ)
    return a.ctypes.data_as(typ)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# --------------------------------------------------------------------------
# kernels, [N, T] layout
# --------------------------------------------------------------------------
def lif_forward(inp, v_init, alpha, subtract, theta, theta_low=None, max_spikes=None, fma=True):
    """cuda/lif_kernels.h:40-93.  Returns (spikes, v_mem) with v_mem before the reset."""
    inp = _f32(inp); N, T = inp.shape
    v_init, alpha, subtract, theta = map(_f32, (v_init, alpha, subtract, theta))
    apply_low = theta_low is not None
    tl = _f32(theta_low) if apply_low else np.zeros(N, np.float32)
    spikes = np.empty_like(inp); vmem = np.empty_like(inp)
    ms = 0xFFFFFFFF if max_spikes is None else int(max_spikes)
    _load(fma).orc_lif_forward(_p(spikes), _p(vmem), _p(inp), _p(v_init), _p(alpha), _p(subtract),
                               _p(theta), _p(tl), ctypes.c_int(int(apply_low)), ctypes.c_uint32(ms),
                               ctypes.c_int64(N), ctypes.c_int64(T))
    return spikes, vmem


def lif_backward(output_grad, surr, not_clipped, alpha, subtract_scaled, fma=True):
    """cuda/lif_kernels.h:122-168 (the O(T^2) double loop)."""
    output_grad, surr, not_clipped = map(_f32, (output_grad, surr, not_clipped))
    alpha, subtract_scaled = _f32(alpha), _f32(subtract_scaled)
    N, T = surr.shape
    gi = np.empty_like(surr)
    _load(fma).orc_lif_backward(_p(gi), _p(output_grad), _p(surr), _p(not_clipped), _p(alpha),
                                _p(subtract_scaled), ctypes.c_int64(N), ctypes.c_int64(T))
    return gi


def lif_backward_alpha(output_grad, vmem_post, v_init, surr, not_clipped, alpha, subtract, fma=True):
    """cuda/lif_kernels.h:199-246."""
    output_grad, vmem_post, surr, not_clipped = map(_f32, (output_grad, vmem_post, surr, not_clipped))
    v_init, alpha, subtract = map(_f32, (v_init, alpha, subtract))
    N, T = surr.shape
    ag = np.empty(N, np.float32)
    _load(fma).orc_lif_backward_alpha(_p(ag), _p(output_grad), _p(vmem_post), _p(v_init), _p(surr),
                                      _p(not_clipped), _p(alpha), _p(subtract),
                                      ctypes.c_int64(N), ctypes.c_int64(T))
    return ag


def leaky_forward(inp, v_init, alpha, fma=True):
    """cuda/leaky_kernels.h:29-58."""
    inp = _f32(inp); N, T = inp.shape
    v_init, alpha = _f32(v_init), _f32(alpha)
    out = np.empty_like(inp)
    _load(fma).orc_leaky_forward(_p(out), _p(inp), _p(v_init), _p(alpha), ctypes.c_int64(N), ctypes.c_int64(T))
    return out


def leaky_backward(output_grad, alpha, fma=True):
    """cuda/leaky_kernels.h:82-110."""
    output_grad = _f32(output_grad); N, T = output_grad.shape
    alpha = _f32(alpha)
    gi = np.empty_like(output_grad)
    _load(fma).orc_leaky_backward(_p(gi), _p(output_grad), _p(alpha), ctypes.c_int64(N), ctypes.c_int64(T))
    return gi


def leaky_backward_alpha(output_grad, output, v_init, alpha, fma=True):
    """cuda/leaky_kernels.h:133-165."""
    output_grad, output = _f32(output_grad), _f32(output)
    v_init, alpha = _f32(v_init), _f32(alpha)
    N, T = output.shape
    ag = np.empty(N, np.float32)
    _load(fma).orc_leaky_backward_alpha(_p(ag), _p(output_grad), _p(output), _p(v_init), _p(alpha),
                                        ctypes.c_int64(N), ctypes.c_int64(T))
    return ag


# --------------------------------------------------------------------------
# double-precision ground truth
# --------------------------------------------------------------------------
def lif_backward_f64(output_grad, surr, not_clipped, alpha, subtract, vmem_post=None, v_init=None):
    """Reverse-time recurrence in double.  Returns (input_grad, alpha_grad | None)."""
    output_grad, surr, not_clipped = map(_f32, (output_grad, surr, not_clipped))
    alpha, subtract = _f32(alpha), _f32(subtract)
    N, T = surr.shape
    gi = np.empty((N, T), np.float64)
    want_alpha = vmem_post is not None
    ag = np.empty(N, np.float64) if want_alpha else None
    vp = _f32(vmem_post) if want_alpha else None
    vi = _f32(v_init) if want_alpha else None
    _load().orc_lif_backward_f64(_p(gi, _f64p), _p(ag, _f64p), _p(output_grad), _p(surr), _p(not_clipped),
                                 _p(vp), _p(vi), _p(alpha), _p(subtract),
                                 ctypes.c_int64(N), ctypes.c_int64(T))
    return gi, ag


def leaky_forward_f64(inp, v_init, alpha):
    inp = _f32(inp); N, T = inp.shape
    out = np.empty((N, T), np.float64)
    _load().orc_leaky_forward_f64(_p(out, _f64p), _p(inp), _p(_f32(v_init)), _p(_f32(alpha)),
                                  ctypes.c_int64(N), ctypes.c_int64(T))
    return out


def leaky_backward_f64(output_grad, alpha, inp=None, v_init=None):
    output_grad = _f32(output_grad); N, T = output_grad.shape
    gi = np.empty((N, T), np.float64)
    want_alpha = inp is not None
    ag = np.empty(N, np.float64) if want_alpha else None
    _load().orc_leaky_backward_f64(_p(gi, _f64p), _p(ag, _f64p), _p(output_grad),
                                   _p(_f32(inp) if want_alpha else None),
                                   _p(_f32(v_init) if want_alpha else None), _p(_f32(alpha)),
                                   ctypes.c_int64(N), ctypes.c_int64(T))
    return gi, ag


def lif_forward_ext(inp, v_init, alpha, subtract, theta, theta_low=None, max_spikes=None, in_scale=None,
                    reset_to_value=False):
    """cuda/lif_kernels.h:40-93 plus the two options of the B200 library: a per-neuron input scale (its product
    with the input is rounded before the fused multiply-add, as a separate PyTorch multiplication in front of
    the kernel gives, layers/lif.py:206-209) and "reset to `subtract` where a spike occurred" instead of
    "subtract per spike" (not a reference mode).  Returns (spikes, v_mem)."""
    inp = _f32(inp); N, T = inp.shape
    v_init, alpha, subtract, theta = map(_f32, (v_init, alpha, subtract, theta))
    apply_low = theta_low is not None
    tl = _f32(theta_low) if apply_low else np.zeros(N, np.float32)
    sc = None if in_scale is None else _f32(in_scale)
    spikes = np.empty_like(inp); vmem = np.empty_like(inp)
    ms = 0xFFFFFFFF if max_spikes is None else int(max_spikes)
    _load().orc_lif_forward_ext(_p(spikes), _p(vmem), _p(inp), _p(v_init), _p(alpha), _p(subtract), _p(theta),
                                _p(tl), ctypes.c_int(int(apply_low)), ctypes.c_uint32(ms), _p(sc),
                                ctypes.c_int(int(bool(reset_to_value))), ctypes.c_int64(N), ctypes.c_int64(T))
    return spikes, vmem


def _f64(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float64)


def lif_syn_backward_f64(grad_spikes, v_mem, spikes, i_syn, inp, surr, v_init, i_init, alpha_syn, scale_syn,
                         scale_mem, alpha_mem, subtract, theta_low=None, reset_to_value=False, grad_v_mem=None,
                         grad_v_last=None, grad_i_syn=None, grad_i_last=None):
    """Float64 adjoint of the layer chain leaky -> scale -> spike step (layers/lif.py:185-258) linearised at the
    given forward results; see orc_lif_syn_backward_f64.  All per-neuron arguments hold N values.

    Returns dict(grad_input, grad_alpha_mem, grad_scale_mem, grad_alpha_syn, grad_scale_syn, grad_v_init,
    grad_i_init), float64.
    """
    v_mem = _f64(v_mem); N, T = v_mem.shape
    full = lambda a: None if a is None else _f64(a)
    per_n = lambda a: _f64(np.broadcast_to(np.asarray(a, np.float64), (N,)))
    args = dict(go=_f64(grad_spikes), gv=full(grad_v_mem), gvl=None if grad_v_last is None else per_n(grad_v_last),
                gis=full(grad_i_syn), gil=None if grad_i_last is None else per_n(grad_i_last),
                v=v_mem, a=_f64(spikes), i=_f64(i_syn), x=_f64(inp), s=_f64(surr),
                v0=per_n(v_init), i0=per_n(i_init), as_=per_n(alpha_syn), ss=per_n(scale_syn), sm=per_n(scale_mem),
                am=per_n(alpha_mem), c=per_n(subtract), lo=None if theta_low is None else per_n(theta_low))
    out = {k: np.empty(N, np.float64) for k in ("grad_alpha_mem", "grad_scale_mem", "grad_alpha_syn", "grad_scale_syn",
                                                "grad_v_init", "grad_i_init")}
    out["grad_input"] = np.empty((N, T), np.float64)
    d = lambda a: _p(a, _f64p)
    _load().orc_lif_syn_backward_f64(
        d(out["grad_input"]), d(out["grad_alpha_mem"]), d(out["grad_scale_mem"]), d(out["grad_alpha_syn"]),
        d(out["grad_scale_syn"]), d(out["grad_v_init"]), d(out["grad_i_init"]),
        d(args["go"]), d(args["gv"]), d(args["gvl"]), d(args["gis"]), d(args["gil"]),
        d(args["v"]), d(args["a"]), d(args["i"]), d(args["x"]), d(args["s"]), d(args["v0"]), d(args["i0"]),
        d(args["as_"]), d(args["ss"]), d(args["sm"]), d(args["am"]), d(args["c"]), d(args["lo"]),
        ctypes.c_int(int(bool(reset_to_value))), ctypes.c_int64(N), ctypes.c_int64(T))
    return out


def surrogate_f64(kind: str, v, theta, p0, p1=1.0):
    """The three closed-form surrogates evaluated in float64 (ground truth for the fused kernels).
    kind: "single_exponential" (p0 = grad_width, p1 = grad_scale), "heaviside" (p0 = window),
    "periodic_exponential" (p0 = grad_width, p1 = grad_scale)."""
    v = np.asarray(v, np.float64); th = np.asarray(theta, np.float64)
    if kind == "single_exponential":
        w = th * p0
        return p1 / w * np.exp(-np.abs(v - th) / w)
    if kind == "heaviside":
        return (v >= th - p0).astype(np.float64) / th
    if kind == "periodic_exponential":
        half = th / 2.0
        u = v - half
        w = np.where(v >= th, u - np.floor(u / th), u)
        return p1 * np.exp(-np.abs(w - half) / p0) / th
    raise ValueError(kind)


# --------------------------------------------------------------------------
# surrogate gradients (this project's definitions; float32 numpy)
# --------------------------------------------------------------------------
def surrogate_single_exponential(v, theta, grad_width=0.5, grad_scale=1.0):
    """s = grad_scale / w * exp(-|v - theta| / w),  w = grad_width * theta."""
    v = _f32(v); theta = _f32(theta)
    w = (theta * np.float32(grad_width)).astype(np.float32)
    return (np.float32(grad_scale) / w * np.exp(-np.abs(v - theta) / w)).astype(np.float32)


def surrogate_heaviside(v, theta, window=1.0):
    """s = [v >= theta - window] / theta."""
    v = _f32(v); theta = _f32(theta)
    return ((v >= (theta - np.float32(window))).astype(np.float32) / theta).astype(np.float32)


def surrogate_periodic_exponential(v, theta, grad_width=0.5, grad_scale=1.0):
    """Exponential bump repeated with period theta above threshold.

    u = v - theta/2;  below threshold w = u, at or above it w = u - floor(u / theta);
    s = grad_scale * exp(-|w - theta/2| / grad_width) / theta.
    """
    v = _f32(v); theta = _f32(theta)
    half = (theta / np.float32(2.0)).astype(np.float32)
    u = (v - half).astype(np.float32)
    per = (u - np.floor(u / theta)).astype(np.float32)
    w = np.where(v >= theta, per, u).astype(np.float32)
    return (np.float32(grad_scale) * np.exp(-np.abs(w - half) / np.float32(grad_width)) / theta).astype(np.float32)


# --------------------------------------------------------------------------
# Function-level glue
# --------------------------------------------------------------------------
def integrate_and_fire_backward(grad_output, grad_v_mem, v_mem, spikes, v_init, alpha, subtract, theta,
                                theta_low, surrogate_fn: Callable, want_alpha_grad: bool, fma=True):
    """sinabs/exodus/spike.py:229-291 with numpy in place of torch.

    Returns (grad_input, grad_alpha | None, grad_init).
    """
    v_mem = _f32(v_mem)
    theta = _f32(theta); alpha = _f32(alpha); subtract = _f32(subtract)
    surr = _f32(surrogate_fn(v_mem, theta[:, None]))                    # spike.py:251
    if theta_low is not None:                                            # spike.py:254-257
        not_clipped = (v_mem > _f32(theta_low)[:, None]).astype(np.float32)
    else:
        not_clipped = np.ones_like(surr)
    g = (surr * _f32(grad_output)).astype(np.float32) + _f32(grad_v_mem)  # spike.py:266
    grad_input = lif_backward(g, surr, not_clipped, alpha, (alpha * subtract).astype(np.float32), fma=fma)
    grad_alpha = None
    if want_alpha_grad:                                                  # spike.py:273-283
        v_post = (v_mem - subtract[:, None] * _f32(spikes)).astype(np.float32)
        grad_alpha = lif_backward_alpha(g, v_post, v_init, surr, not_clipped, alpha, subtract, fma=fma)
    grad_init = (alpha * grad_input[:, 0]).astype(np.float32)            # spike.py:289
    return grad_input, grad_alpha, grad_init


def leaky_integrator_backward(grad_output, out, v_init, alpha, want_alpha_grad: bool, fma=True):
    """sinabs/exodus/leaky.py:53-76.  Returns (grad_input, grad_alpha | None, grad_init)."""
    alpha = _f32(alpha)
    grad_alpha = leaky_backward_alpha(grad_output, out, v_init, alpha, fma=fma) if want_alpha_grad else None
    grad_input = leaky_backward(grad_output, alpha, fma=fma)
    return grad_input, grad_alpha, (alpha * grad_input[:, 0]).astype(np.float32)
