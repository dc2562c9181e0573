"""Leaky-integrator autograd Functions.

``LeakyIntegrator`` keeps the signature, validation and return values of the
reference Function (``sinabs/exodus/leaky.py:5-76``) on ``[N, T]`` tensors.
``LeakyIntegratorTM`` is the same recurrence on a layer's time-major
``(B, T, M)`` tensor with un-expanded parameters and a fused input scale.

Forward is one launch of ``exb_leaky_forward``; backward one launch of
``exb_leaky_backward`` (input gradient, alpha gradient, scale gradient and
``grad_init`` in the same reverse sweep).
"""
from __future__ import annotations

import torch

from . import _lib
from .spike import _flat32, _fold_decay_grad, _mode_of, _reduce_to_param

# Below this many 128-neuron tiles the sequential kernels cannot give every SM a CTA, and the
# time axis is split instead (exb_leaky_*_scan).
_SCAN_MAX_TILES = 148


# Scan workspaces, one per (device, stream, size), zeroed when made.  A scan call that runs to its end leaves
# its workspace zeroed again, so launches that follow one another on a stream share one and need no memset
# (`clean`).  Tensors made during a CUDA-graph capture belong to the graph's pool and are not kept.
_SCAN_WS: dict = {}


def _scan_workspace(B: int, T: int, M: int, layout: int, device):
    """(scratch tensor, clean) for the time-parallel scan, or (None, False) when the plain kernels are the better choice."""
    if layout != _lib.LAYOUT_BTM or B * ((M + 127) // 128) >= _SCAN_MAX_TILES:
        return None, False
    nbytes = _lib.leaky_scan_workspace_bytes(B, T, M)
    if nbytes <= 0:
        return None, False
    words = (nbytes + 3) // 4
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(words, dtype=torch.int32, device=device), False
    key = (str(device), torch.cuda.current_stream(device).cuda_stream, words)
    ws = _SCAN_WS.get(key)
    if ws is None:
        if len(_SCAN_WS) >= 64:
            _SCAN_WS.clear()
        ws = _SCAN_WS[key] = torch.zeros(words, dtype=torch.int32, device=device)
    return ws, True


class _LeakyCore:
    @staticmethod
    def forward(ctx, inp, alpha, v_init, in_scale, B, T, M, layout, total=None, decay_flags=0, scale_flags=0, acc=None):
        """``decay_flags`` / ``scale_flags`` / ``acc``: as in the spiking Functions (``spike._LifCore.forward``)."""
        N = B * M
        a_f, sc_f, vi_f = _flat32(alpha), _flat32(in_scale), _flat32(v_init)
        modes = dict(alpha=_mode_of(a_f, M, N, "alpha") | decay_flags, scale=_mode_of(sc_f, M, N, "in_scale") | scale_flags)
        out = torch.empty_like(inp)
        if T == 0:      # nothing to integrate: the state passes through unchanged
            v_last = vi_f.clone() if vi_f is not None else torch.zeros(N, dtype=torch.float32, device=inp.device)
        else:
            v_last = torch.empty(N, dtype=torch.float32, device=inp.device)
        ws, clean = _scan_workspace(B, T, M, layout, inp.device) if T > 0 else (None, False)
        if ws is not None:
            _lib.leaky_forward_scan(out, inp, vi_f, (a_f, modes["alpha"]), (sc_f, modes["scale"]), v_last, ws, B, T, M,
                                    out_sum=total, clean=clean)
        else:
            _lib.leaky_forward(out, inp, vi_f, (a_f, modes["alpha"]), (sc_f, modes["scale"]), v_last, B, T, M, layout,
                               out_sum=total)
        ctx.set_materialize_grads(False)
        ctx.geometry = (B, T, M, layout)
        ctx.modes = modes
        ctx.want_alpha = alpha.requires_grad
        ctx.scale_derived = bool(scale_flags)
        ctx.want_scale = (in_scale is not None and in_scale.requires_grad) or (ctx.scale_derived and ctx.want_alpha)
        ctx.flags = (decay_flags, scale_flags)
        ctx.acc = acc if (ctx.want_alpha and acc is not None and not (in_scale is not None and in_scale.requires_grad)) else None
        ctx.alpha_shape = alpha.shape
        ctx.scale_shape = None if in_scale is None else in_scale.shape
        ctx.v_init_shape = None if v_init is None else v_init.shape
        ctx.has = (sc_f is not None, vi_f is not None)
        saved = [a_f] + [t for t in (sc_f, vi_f) if t is not None]
        if ctx.want_alpha:
            saved.append(out)
        if ctx.want_scale:
            saved.append(inp)
        ctx.save_for_backward(*saved)
        return out, v_last

    @staticmethod
    def backward(ctx, grad_out, grad_v_last):
        B, T, M, layout = ctx.geometry
        N = B * M
        saved = list(ctx.saved_tensors)
        a_f = saved.pop(0)
        sc_f = saved.pop(0) if ctx.has[0] else None
        vi_f = saved.pop(0) if ctx.has[1] else None
        out = saved.pop(0) if ctx.want_alpha else None
        inp = saved.pop(0) if ctx.want_scale else None
        dev = a_f.device
        if grad_out is None:
            shape = (N, T) if layout == _lib.LAYOUT_NT else (B, T, M)
            grad_out = torch.zeros(shape, dtype=torch.float32, device=dev)
        grad_out = grad_out.contiguous()
        if grad_v_last is not None:
            grad_v_last = grad_v_last.to(torch.float32).reshape(-1).contiguous()
        new = torch.zeros if T == 0 else torch.empty      # an empty sweep launches nothing
        grad_input = torch.empty_like(grad_out)
        grad_init = new(N, dtype=torch.float32, device=dev) if ctx.v_init_shape is not None else None
        ws, clean = _scan_workspace(B, T, M, layout, dev) if T > 0 else (None, False)
        modes = ctx.modes
        decay_flags, scale_flags = ctx.flags
        shape_mode = modes["alpha"] & _lib.PARAM_SHAPE_MASK

        def launch(ga, gs, acc):
            if ws is not None:
                _lib.leaky_backward_scan(grad_input, ga, grad_init, gs, grad_out, grad_v_last, out, inp, vi_f,
                                         (a_f, modes["alpha"]), (sc_f, modes["scale"]), ws, B, T, M, acc_decay=acc,
                                         clean=clean)
                return True
            return _lib.leaky_backward(grad_input, ga, grad_init, gs, grad_out, grad_v_last, out, inp, vi_f,
                                       (a_f, modes["alpha"]), (sc_f, modes["scale"]), B, T, M, layout, acc_decay=acc)

        if ctx.acc is not None and T > 0 and launch(None, None, ctx.acc):
            grad_alpha = torch.empty(a_f.numel(), dtype=torch.float32, device=dev)
            _lib.acc_finish(grad_alpha, ctx.acc)
            grad_alpha = grad_alpha.reshape(ctx.alpha_shape)
            grad_scale = None
        else:
            ga = new(N, dtype=torch.float32, device=dev) if ctx.want_alpha else None
            gs = new(N, dtype=torch.float32, device=dev) if ctx.want_scale else None
            launch(ga, gs, None)
            grad_alpha = _reduce_to_param(ga, ctx.alpha_shape, shape_mode, B, M) if ctx.want_alpha else None
            grad_scale = None
            if ctx.want_scale and not ctx.scale_derived:
                grad_scale = _reduce_to_param(gs, ctx.scale_shape, modes["scale"] & _lib.PARAM_SHAPE_MASK, B, M)
            if ctx.want_alpha and (decay_flags or ctx.scale_derived):
                gs_p = _reduce_to_param(gs, ctx.alpha_shape, shape_mode, B, M) if ctx.scale_derived else None
                grad_alpha = _fold_decay_grad(grad_alpha, gs_p, a_f.reshape(ctx.alpha_shape), decay_flags, scale_flags,
                                              None if sc_f is None else sc_f.reshape(-1))
        if grad_init is not None:
            grad_init = grad_init.reshape(ctx.v_init_shape)
        return grad_input, grad_alpha, grad_init, grad_scale


class LeakyIntegrator(torch.autograd.Function):
    """Drop-in for the reference ``LeakyIntegrator``: ``apply(inp, alpha, v_mem_init) -> out`` on ``[N, T]``."""

    @staticmethod
    def forward(ctx, inp, alpha, v_mem_init):
        if not inp.ndim == 2:
            raise ValueError("'inp' must be 2D, (N, Time)")
        if not inp.is_contiguous():
            raise ValueError("'inp' has to be contiguous.")
        if not alpha.ndim == 1:
            raise ValueError("'alpha' must be 1D, (N,)")
        if not alpha.is_contiguous():
            raise ValueError("'alpha' has to be contiguous.")
        if not v_mem_init.ndim == 1:
            raise ValueError("'v_mem_init' must be 1D, (N,)")
        if not v_mem_init.is_contiguous():
            raise ValueError("'v_mem_init' has to be contiguous.")
        N, T = inp.shape
        if alpha.numel() != N or v_mem_init.numel() != N:
            raise ValueError(f"'alpha' and 'v_mem_init' must have one element per row of 'inp' ({N})")
        out, _ = _LeakyCore.forward(ctx, inp, alpha, v_mem_init, None, 1, T, N, _lib.LAYOUT_NT)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        grad_input, grad_alpha, grad_init, _ = _LeakyCore.backward(ctx, grad_output, None)
        return grad_input, grad_alpha, grad_init


class LeakyIntegratorTM(torch.autograd.Function):
    """Leaky integrator on a time-major ``(B, T, M)`` tensor.

    ``apply(inp, alpha, v_init, in_scale, total=None) -> (out, v_last)``; parameters hold
    1, M or B*M values.  ``v_last`` (B*M,) equals ``out[:, -1]`` and carries its own
    gradient, so that keeping the state for the next call costs no full-size tensor.
    ``total``: optional float64 tensor of one element, zeroed by the caller, to which the
    kernel adds ``out.sum()`` (no gradient flows through it).
    """

    @staticmethod
    def forward(ctx, inp, alpha, v_init, in_scale, total=None, decay_flags=0, scale_flags=0, acc=None):
        if inp.ndim != 3:
            raise ValueError("'inp' must be 3D, (batch, time, neurons)")
        if not inp.is_contiguous():
            raise ValueError("'inp' has to be contiguous.")
        B, T, M = inp.shape
        if v_init is not None and v_init.numel() != B * M:
            raise ValueError("'v_init' must hold one value per batch item and neuron")
        return _LeakyCore.forward(ctx, inp, alpha, v_init, in_scale, B, T, M, _lib.LAYOUT_BTM, total, decay_flags,
                                  scale_flags, acc)

    @staticmethod
    def backward(ctx, grad_out, grad_v_last):
        return _LeakyCore.backward(ctx, grad_out, grad_v_last) + (None, None, None, None)
