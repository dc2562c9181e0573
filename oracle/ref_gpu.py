"""Runs the REFERENCE's own CUDA kernels (``oracle/_ref/libexodus_ref.so``).  Test infrastructure only.

The library is built by ``oracle/build.py`` from the reference checkout and is
present only where that build ran.  The functions here take float32 CUDA
tensors in the reference's ``[N, T]`` layout and restate, with PyTorch ops, the
glue of the reference's autograd Functions around each kernel
(``sinabs/exodus/spike.py:193-212,251-289``, ``leaky.py:43-72``).
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, Optional

import torch

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libexodus_ref.so")
_lib = None
_vp, _i, _u = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint


def available() -> bool:
    return os.path.exists(_PATH)


def _load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(_PATH)
        lib.ref_sync.restype = _i
        lib.ref_lif_forward.argtypes = [_vp] * 8 + [_i, _i, _u, _u]
        lib.ref_lif_backward.argtypes = [_vp] * 6 + [_u, _u]
        lib.ref_lif_backward_alpha.argtypes = [_vp] * 8 + [_u, _u]
        lib.ref_leaky_forward.argtypes = [_vp] * 4 + [_u, _u]
        lib.ref_leaky_backward.argtypes = [_vp] * 3 + [_u, _u]
        lib.ref_leaky_backward_alpha.argtypes = [_vp] * 5 + [_u, _u]
        _lib = lib
    return _lib


def _sync():
    rc = _load().ref_sync()
    if rc != 0:
        raise RuntimeError(f"reference kernel failed (code {rc})")


def _c(t: torch.Tensor) -> torch.Tensor:
    assert t.is_cuda and t.dtype == torch.float32
    return t.contiguous()


def lif_forward(inp, v_init, alpha, subtract, theta, theta_low=None, max_spikes=None):
    """spike.py:193-207 -> lifForward.  Returns (spikes, v_mem)."""
    inp = _c(inp); N, T = inp.shape
    apply_low = theta_low is not None
    tl = _c(theta_low) if apply_low else torch.empty_like(theta)
    spikes = torch.empty_like(inp); v_mem = torch.empty_like(inp)
    torch.cuda.synchronize()
    _load().ref_lif_forward(spikes.data_ptr(), v_mem.data_ptr(), inp.data_ptr(), _c(v_init).data_ptr(),
                            _c(alpha).data_ptr(), _c(subtract).data_ptr(), _c(theta).data_ptr(), tl.data_ptr(),
                            int(apply_low), -1 if max_spikes is None else int(max_spikes), N, T)
    _sync()
    return spikes, v_mem


def lif_backward_kernels(g, surr, not_clipped, alpha, subtract, v_post=None, v_init=None):
    """lifBackward (+ lifBackwardAlpha when v_post is given) on prepared tensors."""
    surr = _c(surr); N, T = surr.shape
    g = _c(g); nc = _c(not_clipped); alpha = _c(alpha); subtract = _c(subtract)
    cp = (alpha * subtract).contiguous()
    gi = torch.empty_like(surr)
    torch.cuda.synchronize()
    _load().ref_lif_backward(gi.data_ptr(), g.data_ptr(), surr.data_ptr(), nc.data_ptr(), alpha.data_ptr(),
                             cp.data_ptr(), N, T)
    ga = None
    if v_post is not None:
        ga = torch.empty_like(alpha)
        vp = _c(v_post); vi = _c(v_init)
        _load().ref_lif_backward_alpha(ga.data_ptr(), g.data_ptr(), vp.data_ptr(), vi.data_ptr(), surr.data_ptr(),
                                       nc.data_ptr(), alpha.data_ptr(), subtract.data_ptr(), N, T)
    _sync()
    return gi, ga


def integrate_and_fire_backward(grad_output, grad_v_mem, v_mem, spikes, v_init, alpha, subtract, theta,
                                theta_low, surrogate_fn: Callable, want_alpha_grad: bool):
    """spike.py:229-291.  Returns (grad_input, grad_alpha | None, grad_init, surr, not_clipped, g)."""
    surr = surrogate_fn(v_mem, theta.unsqueeze(1)).contiguous()
    if theta_low is not None:
        not_clipped = (v_mem > theta_low.unsqueeze(1)).float()
    else:
        not_clipped = torch.ones_like(surr)
    g = surr * grad_output.contiguous() + grad_v_mem.contiguous()
    v_post = (v_mem - subtract.unsqueeze(1) * spikes) if want_alpha_grad else None
    gi, ga = lif_backward_kernels(g, surr, not_clipped, alpha, subtract, v_post, v_init)
    return gi, ga, alpha * gi[:, 0], surr, not_clipped, g


def leaky_forward(inp, v_init, alpha):
    inp = _c(inp); N, T = inp.shape
    out = torch.empty_like(inp)
    torch.cuda.synchronize()
    _load().ref_leaky_forward(out.data_ptr(), inp.data_ptr(), _c(v_init).data_ptr(), _c(alpha).data_ptr(), N, T)
    _sync()
    return out


def leaky_backward(grad_output, alpha, out=None, v_init=None):
    """leaky.py:53-72.  Returns (grad_input, grad_alpha | None, grad_init)."""
    go = _c(grad_output); N, T = go.shape
    alpha = _c(alpha)
    gi = torch.empty_like(go)
    ga = None
    torch.cuda.synchronize()
    if out is not None:
        ga = torch.empty_like(alpha)
        _load().ref_leaky_backward_alpha(ga.data_ptr(), go.data_ptr(), _c(out).data_ptr(), _c(v_init).data_ptr(),
                                         alpha.data_ptr(), N, T)
    _load().ref_leaky_backward(gi.data_ptr(), go.data_ptr(), alpha.data_ptr(), N, T)
    _sync()
    return gi, ga, alpha * gi[:, 0]
