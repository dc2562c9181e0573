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
