"""Spiking autograd Functions.

``IntegrateAndFire`` keeps the signature, validation, return values and error
types of the reference Function (``sinabs/exodus/spike.py:107-291``) and runs on
``[N, T]`` tensors.  ``IntegrateAndFireTM`` is the same computation on a layer's
own time-major ``(B, T, M)`` tensor with un-expanded parameters; the layers use it
so that no transpose or parameter broadcast is ever materialised.

Forward is one launch of ``exb_lif_forward``.  Backward is one launch of
``exb_lif_backward``, which replaces the reference's surrogate evaluation, clip
mask, gradient combination, ``lifBackward``, ``lifBackwardAlpha`` and
``grad_init`` (``spike.py:251-289``).
"""
from __future__ import annotations

import os
import weakref
from typing import Callable, Optional, Tuple

import torch

from . import _lib
from .surrogate import classify


def _mode_of(t: Optional[torch.Tensor], M: int, N: int, name: str) -> int:
    if t is None:
        return _lib.PARAM_SCALAR
    k = t.numel()
    if k == 1:
        return _lib.PARAM_SCALAR
    if k == M:
        return _lib.PARAM_PER_M
    if k == N:
        return _lib.PARAM_PER_N
    raise ValueError(f"'{name}' has {k} elements; expected 1, {M} (per neuron) or {N} (per batch item and neuron)")


def _reduce_to_param(per_instance: torch.Tensor, shape, mode: int, B: int, M: int) -> torch.Tensor:
    """Sum a per-instance (N,) gradient down to the parameter's own shape."""
    if mode == _lib.PARAM_PER_N:
        g = per_instance
    elif mode == _lib.PARAM_PER_M:
        g = per_instance.view(B, M).sum(0)
    else:
        g = per_instance.sum()
    return g.reshape(shape)


def _fold_decay_grad(ga: torch.Tensor, gs: Optional[torch.Tensor], raw: torch.Tensor, decay_flags: int,
                     scale_flags: int, given_scale: Optional[torch.Tensor]) -> torch.Tensor:
    """PyTorch form of what the kernels' float64 accumulator holds, for shapes the reducing kernels do not take:
    the gradient w.r.t. the decay values as passed (alpha, or tau with ``PARAM_IS_TAU``) from the per-instance
    gradients w.r.t. alpha (``ga``) and w.r.t. a scale derived from alpha (``gs``), already reduced to the
    parameter's shape."""
    alpha = torch.exp(-torch.reciprocal(raw)) if decay_flags & _lib.PARAM_IS_TAU else raw
    g = ga
    if gs is not None:
        om, ta = scale_flags & _lib.SCALE_ONE_MINUS_ALPHA, scale_flags & _lib.SCALE_TIMES_ALPHA
        if om and ta:
            g = g + (1.0 - 2.0 * alpha) * gs
        elif om:
            g = g - gs
        elif ta:
            g = g + (gs if given_scale is None else given_scale * gs)
    if decay_flags & _lib.PARAM_IS_TAU:
        r = torch.reciprocal(raw)
        g = g * alpha * r * r
    return g


def acc_eligible(inp: torch.Tensor) -> bool:
    """Whether the backward kernels that reduce parameter gradients in the kernel take this (B, T, M) tensor (the
    TMA-staged family: neurons % 4 == 0, 16-byte aligned contiguous float32 storage)."""
    return (inp.ndim == 3 and inp.is_cuda and inp.dtype == torch.float32 and inp.is_contiguous()
            and inp.shape[2] % 4 == 0 and inp.data_ptr() % 16 == 0 and inp.numel() > 0
            and inp.shape[1] * inp.shape[2] < 2 ** 31 and os.environ.get("EXB_DISABLE_TMA", "0") != "1")


def _flat32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """Detached flat float32 view (or copy) of a parameter, as the library takes it.  The common cases -- a constant
    that is already such a vector, a flat float32 parameter -- cost no or one tensor operation."""
    if t is None:
        return None
    if t.dtype == torch.float32 and t.dim() == 1 and t.is_contiguous():
        return t.detach() if t.requires_grad else t
    return t.detach().to(torch.float32).reshape(-1).contiguous()


class _LifCore:
    """Shared forward/backward bodies; ``layout`` decides how (B, T, M) maps to memory."""

    @staticmethod
    def forward(ctx, inp, alpha, v_init, theta, subtract, min_v_mem, in_scale, surrogate_fn, max_spikes,
                reset_mode, spike_count, B, T, M, layout, scale_grad_from_state=False, record=None,
                decay_flags=0, scale_flags=0, acc=None, recompute=False, keep_v_mem=True):
        """``decay_flags`` / ``scale_flags``: ``PARAM_IS_TAU`` and ``SCALE_*`` bits for the alpha and scale arguments
        (the kernels then derive alpha = exp(-1/tau) and the scale from alpha; the gradient returned for ``alpha`` is
        the one w.r.t. the values passed, scale part included).  ``acc``: zeroed float64 tensor shaped like the
        flattened ``alpha`` that the backward kernel reduces that gradient into (no per-instance vector, no
        reduction or chain-rule launches).  ``recompute`` (time-major layout, built-in surrogates, no ``record``): keep
        the input and one checkpoint of the state per ``CKPT_EVERY`` steps instead of ``v_mem``; the backward kernel
        rebuilds ``v_mem`` bit for bit.  The second result is then ``None``.  Shapes the checkpointing kernels do not
        take fall back to the ordinary pair.  ``keep_v_mem=False`` (a call that is neither differentiated nor recorded):
        ``v_mem`` is not written at all where the kernels allow it (second result ``None``)."""
        N = B * M
        a_f, th_f, c_f, lo_f, sc_f = map(_flat32, (alpha, theta, subtract, min_v_mem, in_scale))
        modes = dict(
            alpha=_mode_of(a_f, M, N, "alpha") | decay_flags, theta=_mode_of(th_f, M, N, "threshold"),
            subtract=_mode_of(c_f, M, N, "membrane_subtract"), lo=_mode_of(lo_f, M, N, "min_v_mem"),
            scale=_mode_of(sc_f, M, N, "in_scale") | scale_flags)
        vi_f = _flat32(v_init)
        spikes = torch.empty_like(inp)
        if T == 0:      # nothing to integrate: the state passes through unchanged
            v_post_last = vi_f.clone() if vi_f is not None else torch.zeros(N, dtype=torch.float32, device=inp.device)
        else:
            v_post_last = torch.empty(N, dtype=torch.float32, device=inp.device)
        ckpt = None
        if (recompute and layout == _lib.LAYOUT_BTM and record is None and acc_eligible(inp)
                and classify(surrogate_fn)[0] != _lib.SURR_GENERIC):
            ckpt = torch.empty(_lib.ckpt_shape(B, T, M), dtype=torch.float32, device=inp.device)
            if not _lib.lif_forward_ckpt(spikes, ckpt, inp, vi_f, (sc_f, modes["scale"]), (a_f, modes["alpha"]),
                                         (c_f, modes["subtract"]), (th_f, modes["theta"]), (lo_f, modes["lo"]),
                                         max_spikes, reset_mode, v_post_last, spike_count, B, T, M):
                ckpt = None
        v_mem = None
        params = ((sc_f, modes["scale"]), (a_f, modes["alpha"]), (c_f, modes["subtract"]), (th_f, modes["theta"]),
                  (lo_f, modes["lo"]), max_spikes, reset_mode, v_post_last, spike_count, B, T, M, layout)
        done = ckpt is not None
        if not done and not keep_v_mem and layout == _lib.LAYOUT_BTM and record is None and T > 0:
            done = _lib.lif_forward(spikes, None, inp, vi_f, *params)
        if not done:
            v_mem = torch.empty_like(inp)
            _lib.lif_forward(spikes, v_mem, inp, vi_f, *params, v_post=record)
        ctx.set_materialize_grads(False)
        ctx.geometry = (B, T, M, layout)
        ctx.modes = modes
        ctx.surrogate_fn = surrogate_fn
        ctx.max_spikes = max_spikes
        ctx.reset_mode = reset_mode
        ctx.want_alpha = alpha is not None and alpha.requires_grad
        ctx.scale_derived = bool(scale_flags)
        # a scale derived from alpha sends its gradient to alpha; a separate scale tensor gets its own
        ctx.want_scale = (in_scale is not None and in_scale.requires_grad) or (ctx.scale_derived and ctx.want_alpha)
        ctx.flags = (decay_flags, scale_flags)
        ctx.acc = acc if (ctx.want_alpha and acc is not None and not (in_scale is not None and in_scale.requires_grad)) else None
        # The scale gradient either reads the forward input again or is rebuilt from v_mem alone
        # (no extra tensor kept alive or streamed); the latter needs every scale to be non-zero.
        ctx.save_input = (ctx.want_scale and not scale_grad_from_state) or ckpt is not None
        ctx.recompute = ckpt is not None
        ctx.alpha_shape = None if alpha is None else alpha.shape
        ctx.scale_shape = None if in_scale is None else in_scale.shape
        ctx.v_init_shape = None if v_init is None else v_init.shape
        ctx.has = tuple(t is not None for t in (c_f, lo_f, sc_f, vi_f))
        if ckpt is None and v_mem is None:      # spikes only: nothing to differentiate
            return spikes, None, v_post_last
        saved = [ckpt if ckpt is not None else v_mem, a_f, th_f]
        saved += [t for t in (c_f, lo_f, sc_f, vi_f) if t is not None]
        if ctx.save_input:
            saved.append(inp)
        ctx.save_for_backward(*saved)
        return spikes, v_mem, v_post_last

    @staticmethod
    def backward(ctx, grad_spikes, grad_v_mem, grad_v_last):
        B, T, M, layout = ctx.geometry
        N = B * M
        saved = list(ctx.saved_tensors)
        v_mem, a_f, th_f = saved[:3]
        rest = saved[3:]
        c_f = rest.pop(0) if ctx.has[0] else None
        lo_f = rest.pop(0) if ctx.has[1] else None
        sc_f = rest.pop(0) if ctx.has[2] else None
        vi_f = rest.pop(0) if ctx.has[3] else None
        inp = rest.pop(0) if ctx.save_input else None
        modes = ctx.modes
        dev = v_mem.device
        if ctx.recompute:
            return _LifCore._backward_recompute(ctx, grad_spikes, grad_v_last, v_mem, inp, a_f, th_f, c_f, lo_f, sc_f, vi_f)

        if grad_spikes is None:
            grad_spikes = torch.zeros_like(v_mem)
        grad_spikes = grad_spikes.contiguous()
        if grad_v_mem is not None:
            grad_v_mem = grad_v_mem.contiguous()
        if grad_v_last is not None:
            grad_v_last = grad_v_last.to(torch.float32).reshape(-1).contiguous()

        kind, p0, p1 = classify(ctx.surrogate_fn)
        surr = None
        if kind == _lib.SURR_GENERIC:
            # Any callable: evaluate it with PyTorch exactly like spike.py:251.
            if layout == _lib.LAYOUT_NT:
                th_b = th_f.reshape(-1, 1) if th_f.numel() > 1 else th_f
            else:
                th_b = th_f if th_f.numel() == 1 else (
                    th_f.view(1, 1, M) if modes["theta"] == _lib.PARAM_PER_M else th_f.view(B, 1, M))
            surr = ctx.surrogate_fn(v_mem, th_b).to(torch.float32).contiguous()

        new = torch.zeros if T == 0 else torch.empty      # an empty sweep launches nothing
        grad_input = torch.empty_like(v_mem)
        grad_init = new(N, dtype=torch.float32, device=dev) if ctx.v_init_shape is not None else None
        args = (grad_spikes, grad_v_mem, grad_v_last, v_mem, surr, vi_f, inp, (sc_f, modes["scale"]),
                (a_f, modes["alpha"]), (c_f, modes["subtract"]), (th_f, modes["theta"]), (lo_f, modes["lo"]),
                ctx.max_spikes, ctx.reset_mode, kind, p0, p1, B, T, M, layout)
        decay_flags, scale_flags = ctx.flags
        shape_mode = modes["alpha"] & _lib.PARAM_SHAPE_MASK
        if ctx.acc is not None and T > 0 and _lib.lif_backward(grad_input, None, grad_init, None, *args, acc_decay=ctx.acc):
            # reduced over the batch, chain rule applied, in the kernel; one small launch converts and clears
            grad_alpha = torch.empty(a_f.numel(), dtype=torch.float32, device=dev)
            _lib.acc_finish(grad_alpha, ctx.acc)
            grad_alpha = grad_alpha.reshape(ctx.alpha_shape)
            grad_scale = None
        else:
            ga = new(N, dtype=torch.float32, device=dev) if ctx.want_alpha else None
            gs = new(N, dtype=torch.float32, device=dev) if ctx.want_scale else None
            _lib.lif_backward(grad_input, ga, grad_init, gs, *args)
            grad_alpha = grad_scale = None
            if ctx.want_alpha:
                grad_alpha = _reduce_to_param(ga, ctx.alpha_shape, shape_mode, B, M)
            if ctx.want_scale and not ctx.scale_derived:
                grad_scale = _reduce_to_param(gs, ctx.scale_shape, modes["scale"] & _lib.PARAM_SHAPE_MASK, B, M)
            if ctx.want_alpha and (decay_flags or ctx.scale_derived):
                gs_p = _reduce_to_param(gs, ctx.alpha_shape, shape_mode, B, M) if ctx.scale_derived else None
                grad_alpha = _fold_decay_grad(grad_alpha, gs_p, a_f.reshape(ctx.alpha_shape), decay_flags, scale_flags,
                                              None if sc_f is None else sc_f.reshape(-1))
        if grad_init is not None:
            grad_init = grad_init.reshape(ctx.v_init_shape)
        return grad_input, grad_alpha, grad_init, grad_scale


def _backward_recompute(ctx, grad_spikes, grad_v_last, ckpt, inp, a_f, th_f, c_f, lo_f, sc_f, vi_f):
    """Backward of a forward pass made with ``recompute``: ``exb_lif_backward_ckpt`` on (input, checkpoints)."""
    B, T, M, _ = ctx.geometry
    N = B * M
    modes = ctx.modes
    dev = inp.device
    grad_spikes = torch.zeros_like(inp) if grad_spikes is None else grad_spikes.contiguous()
    if grad_v_last is not None:
        grad_v_last = grad_v_last.to(torch.float32).reshape(-1).contiguous()
    kind, p0, p1 = classify(ctx.surrogate_fn)
    grad_input = torch.empty_like(inp)
    grad_init = torch.empty(N, dtype=torch.float32, device=dev) if ctx.v_init_shape is not None else None
    tail = (grad_spikes, grad_v_last, inp, ckpt, vi_f, (sc_f, modes["scale"]), (a_f, modes["alpha"]),
            (c_f, modes["subtract"]), (th_f, modes["theta"]), (lo_f, modes["lo"]), ctx.max_spikes, ctx.reset_mode,
            kind, p0, p1, B, T, M)
    decay_flags, scale_flags = ctx.flags
    shape_mode = modes["alpha"] & _lib.PARAM_SHAPE_MASK
    grad_alpha = grad_scale = None
    if ctx.acc is not None:
        _lib.lif_backward_ckpt(grad_input, None, grad_init, None, *tail, acc_decay=ctx.acc)
        grad_alpha = torch.empty(a_f.numel(), dtype=torch.float32, device=dev)
        _lib.acc_finish(grad_alpha, ctx.acc)
        grad_alpha = grad_alpha.reshape(ctx.alpha_shape)
    else:
        ga = torch.empty(N, dtype=torch.float32, device=dev) if ctx.want_alpha else None
        gs = torch.empty(N, dtype=torch.float32, device=dev) if ctx.want_scale else None
        _lib.lif_backward_ckpt(grad_input, ga, grad_init, gs, *tail)
        if ctx.want_alpha:
            grad_alpha = _reduce_to_param(ga, ctx.alpha_shape, shape_mode, B, M)
        if ctx.want_scale and not ctx.scale_derived:
            grad_scale = _reduce_to_param(gs, ctx.scale_shape, modes["scale"] & _lib.PARAM_SHAPE_MASK, B, M)
        if ctx.want_alpha and (decay_flags or ctx.scale_derived):
            gs_p = _reduce_to_param(gs, ctx.alpha_shape, shape_mode, B, M) if ctx.scale_derived else None
            grad_alpha = _fold_decay_grad(grad_alpha, gs_p, a_f.reshape(ctx.alpha_shape), decay_flags, scale_flags,
                                          None if sc_f is None else sc_f.reshape(-1))
    if grad_init is not None:
        grad_init = grad_init.reshape(ctx.v_init_shape)
    return grad_input, grad_alpha, grad_init, grad_scale


_LifCore._backward_recompute = staticmethod(_backward_recompute)


def _validate_1d(t: torch.Tensor, name: str) -> None:
    if not t.ndim == 1:
        raise ValueError(f"'{name}' must be 1D, (N,)")
    if not t.is_contiguous():
        raise ValueError(f"'{name}' has to be contiguous.")


# Value checks of the reference Function (spike.py:183,190).  Each one reads a result back from the GPU,
# which drains the launch queue, so the verdict is remembered for as long as the very same tensors (object
# and version counter) come back: parameters checked once are not read back again on every call.
_CHECKED: dict = {}


def _check_values(alpha: torch.Tensor, threshold: torch.Tensor, min_v_mem: Optional[torch.Tensor]) -> None:
    tensors = [t for t in (alpha, threshold, min_v_mem) if t is not None]
    key = tuple(id(t) for t in tensors)
    seen = _CHECKED.get(key)
    if seen is not None and all(r() is t and ver == t._version for (r, ver), t in zip(seen, tensors)):
        return      # the same live tensors, unmodified since they passed
    bad_alpha = ((alpha < 0) | (alpha > 1)).any()
    if min_v_mem is not None:
        bad_alpha, bad_low = torch.stack((bad_alpha, (threshold <= min_v_mem).any())).tolist()   # one read-back
    else:
        bad_alpha, bad_low = bool(bad_alpha), False
    if bad_alpha:
        raise ValueError("'alpha' must be between 0 and 1.")
    if bad_low:
        raise ValueError("`threshold` must be greater than `min_v_mem`.")
    if len(_CHECKED) >= 256:
        _CHECKED.clear()
    _CHECKED[key] = [(weakref.ref(t), t._version) for t in tensors]


class IntegrateAndFire(torch.autograd.Function):
    """Drop-in for the reference ``IntegrateAndFire`` (``[N, T]`` tensors, per-row parameters).

    ``apply(inp, alpha, v_mem_init, threshold, membrane_subtract, min_v_mem,
    surrogate_grad_fn, max_num_spikes_per_bin=None) -> (output_spikes, v_mem)``
    with ``v_mem`` the membrane potential before the reset of each step.
    """

    @staticmethod
    def forward(ctx, inp, alpha, v_mem_init, threshold, membrane_subtract, min_v_mem,
                surrogate_grad_fn: Callable, max_num_spikes_per_bin: Optional[int] = None):
        if membrane_subtract is None:                       # spike.py:157-158
            membrane_subtract = torch.ones_like(alpha) * threshold
        apply_min_v_mem = min_v_mem is not None
        if not inp.ndim == 2:
            raise ValueError("'inp' must be 2D, (N, Time)")
        if not inp.is_contiguous():
            raise ValueError("'inp' has to be contiguous.")
        _validate_1d(alpha, "alpha")
        _validate_1d(membrane_subtract, "membrane_subtract")
        _validate_1d(v_mem_init, "v_mem_init")
        _validate_1d(threshold, "threshold")
        if apply_min_v_mem:
            _validate_1d(min_v_mem, "min_v_mem")
        _check_values(alpha, threshold, min_v_mem)
        N, T = inp.shape
        for t, name in ((alpha, "alpha"), (membrane_subtract, "membrane_subtract"),
                        (v_mem_init, "v_mem_init"), (threshold, "threshold")):
            if t.numel() != N:
                raise ValueError(f"'{name}' must have one element per row of 'inp' ({N}), got {t.numel()}")
        spikes, v_mem, _ = _LifCore.forward(
            ctx, inp, alpha, v_mem_init, threshold, membrane_subtract, min_v_mem, None, surrogate_grad_fn,
            max_num_spikes_per_bin, _lib.RESET_SUBTRACT, None, 1, T, N, _lib.LAYOUT_NT)
        return spikes, v_mem

    @staticmethod
    def backward(ctx, grad_output, grad_v_mem):
        grad_input, grad_alpha, grad_init, _ = _LifCore.backward(ctx, grad_output, grad_v_mem, None)
        return grad_input, grad_alpha, grad_init, None, None, None, None, None


class IntegrateAndFireTM(torch.autograd.Function):
    """Spike scan on a time-major ``(B, T, M)`` tensor.

    ``apply(inp, alpha, v_init, threshold, membrane_subtract, min_v_mem, in_scale,
    surrogate_grad_fn, max_num_spikes_per_bin, reset_mode, spike_count)
    -> (spikes, v_mem, v_post_last)``.

    Parameters hold 1, M or B*M values and are read in place.  ``in_scale``
    multiplies the input per neuron.  ``v_post_last`` (B*M,) is the state after the
    last reset; a gradient arriving on it is folded into the sweep.  ``spike_count``
    is an optional zero-initialised int64 tensor of one element that receives the
    total number of spikes.  ``scale_grad_from_state=True`` makes the backward rebuild the
    gradient w.r.t. ``in_scale`` from the saved membrane potential instead of keeping and re-reading
    the input; the caller guarantees that no scale is zero.  ``record``: optional tensor like ``inp`` that
    the same launch fills with the potential after each step's reset (a plain side output, no gradient).
    ``recompute=True`` / ``keep_v_mem=False``: ``v_mem`` is not materialised (second result ``None``); see
    ``_LifCore.forward``.
    """

    @staticmethod
    def forward(ctx, inp, alpha, v_init, threshold, membrane_subtract, min_v_mem, in_scale,
                surrogate_grad_fn, max_num_spikes_per_bin, reset_mode, spike_count, scale_grad_from_state=False,
                record=None, decay_flags=0, scale_flags=0, acc=None, recompute=False, keep_v_mem=True):
        if inp.ndim != 3:
            raise ValueError("'inp' must be 3D, (batch, time, neurons)")
        if not inp.is_contiguous():
            raise ValueError("'inp' has to be contiguous.")
        B, T, M = inp.shape
        if v_init is not None and v_init.numel() != B * M:
            raise ValueError("'v_init' must hold one value per batch item and neuron")
        return _LifCore.forward(ctx, inp, alpha, v_init, threshold, membrane_subtract, min_v_mem, in_scale,
                                surrogate_grad_fn, max_num_spikes_per_bin, reset_mode, spike_count,
                                B, T, M, _lib.LAYOUT_BTM, scale_grad_from_state, record, decay_flags, scale_flags, acc,
                                recompute, keep_v_mem)

    @staticmethod
    def backward(ctx, grad_spikes, grad_v_mem, grad_v_last):
        grad_input, grad_alpha, grad_init, grad_scale = _LifCore.backward(ctx, grad_spikes, grad_v_mem, grad_v_last)
        return (grad_input, grad_alpha, grad_init, None, None, None, grad_scale, None, None, None, None, None, None,
                None, None, None, None, None)


def fused_synaptic_eligible(inp: torch.Tensor) -> bool:
    """Whether ``LIFSynapticTM`` can take this (B, T, M) tensor: the fused kernels stage through TMA,
    which needs M % 4 == 0 and 16-byte aligned, contiguous float32 storage."""
    return (inp.ndim == 3 and inp.is_cuda and inp.dtype == torch.float32 and inp.is_contiguous()
            and inp.shape[2] % 4 == 0 and inp.data_ptr() % 16 == 0 and inp.numel() > 0)


class LIFSynapticTM(torch.autograd.Function):
    """Synaptic leaky integrator and spiking membrane of a LIF layer as one kernel per direction.

    ``apply(inp, alpha_syn, scale_syn, i_init, alpha_mem, scale_mem, v_init, threshold,
    membrane_subtract, min_v_mem, surrogate_grad_fn, max_num_spikes_per_bin, reset_mode, spike_count)
    -> (spikes, v_mem, v_post_last, i_syn, i_last)`` on a time-major ``(B, T, M)`` tensor:

        i_t = alpha_syn * i_{t-1} + scale_syn * inp_t
        v_t, spikes_t = membrane step on scale_mem * i_t      (as ``IntegrateAndFireTM``)

    Replaces the chain ``LeakyIntegrator`` -> ``(1 - alpha) * i_syn`` -> ``IntegrateAndFire`` of the
    reference layer (``layers/lif.py:185-258``) and saves re-reading ``i_syn`` and ``inp``.
    Parameters hold 1, M or B*M values; ``scale_syn`` / ``scale_mem`` may be None (= 1).
    """

    @staticmethod
    def forward(ctx, inp, alpha_syn, scale_syn, i_init, alpha_mem, scale_mem, v_init, threshold, membrane_subtract,
                min_v_mem, surrogate_grad_fn, max_num_spikes_per_bin, reset_mode, spike_count, flags=(0, 0, 0, 0),
                acc=None, keep_states=True):
        """``keep_states=False`` (a call that is neither differentiated nor recorded): ``v_mem`` and ``i_syn`` are not
        written (second and fourth result ``None``).
        ``flags``: (decay_syn, scale_syn, decay_mem, scale_mem) bits (``PARAM_IS_TAU``, ``SCALE_*``) for the four
        parameter arguments.  ``acc``: (acc_mem, acc_syn), zeroed float64 tensors shaped like the flattened
        ``alpha_mem`` / ``alpha_syn``, into which the backward kernel reduces the gradients w.r.t. the values passed
        for the two decays (scale parts included) when neither scale is a tensor of its own."""
        if not fused_synaptic_eligible(inp):
            raise ValueError("'inp' must be a contiguous float32 CUDA tensor (batch, time, neurons) with neurons % 4 == 0")
        B, T, M = inp.shape
        N = B * M
        f = {k: _flat32(t) for k, t in dict(a_syn=alpha_syn, s_syn=scale_syn, a_mem=alpha_mem, s_mem=scale_mem,
                                            th=threshold, c=membrane_subtract, lo=min_v_mem).items()}
        modes = {k: _mode_of(t, M, N, k) for k, t in f.items()}
        modes["a_syn"] |= flags[0]; modes["s_syn"] |= flags[1]; modes["a_mem"] |= flags[2]; modes["s_mem"] |= flags[3]
        vi_f, ii_f = _flat32(v_init), _flat32(i_init)
        spikes = torch.empty_like(inp)
        v_mem = torch.empty_like(inp) if keep_states else None
        i_syn = torch.empty_like(inp) if keep_states else None
        v_post_last = torch.empty(N, dtype=torch.float32, device=inp.device)
        i_last = torch.empty(N, dtype=torch.float32, device=inp.device)
        spec = lambda k: (f[k], modes[k])
        done = _lib.lif_syn_forward(spikes, v_mem, i_syn, inp, vi_f, ii_f, spec("a_syn"), spec("s_syn"), spec("s_mem"),
                                    spec("a_mem"), spec("c"), spec("th"), spec("lo"), max_num_spikes_per_bin, reset_mode,
                                    v_post_last, i_last, spike_count, B, T, M)
        if not done:
            raise _lib.ExodusLibraryError("exb_lif_syn_forward refused a shape that passed the eligibility check")
        if not keep_states:
            return spikes, None, v_post_last, None, i_last
        ctx.set_materialize_grads(False)
        ctx.geometry = (B, T, M)
        ctx.modes = modes
        ctx.keys = [k for k in f if f[k] is not None]
        ctx.surrogate_fn = surrogate_grad_fn
        ctx.max_spikes = max_num_spikes_per_bin
        ctx.reset_mode = reset_mode
        ctx.param_shapes = {k: (None if t is None else t.shape) for k, t in
                            dict(a_syn=alpha_syn, s_syn=scale_syn, a_mem=alpha_mem, s_mem=scale_mem).items()}
        ctx.param_needs = {k: (t is not None and t.requires_grad) for k, t in
                           dict(a_syn=alpha_syn, s_syn=scale_syn, a_mem=alpha_mem, s_mem=scale_mem).items()}
        ctx.want_params = any(ctx.param_needs.values())
        ctx.flags = flags
        own_scale = (scale_syn is not None) or (scale_mem is not None)
        ctx.acc = acc if (acc is not None and ctx.want_params and not own_scale) else None
        ctx.init_shapes = (None if v_init is None else v_init.shape, None if i_init is None else i_init.shape)
        saved = [v_mem] + [f[k] for k in ctx.keys] + [t for t in (vi_f, ii_f) if t is not None]
        ctx.has_init = (vi_f is not None, ii_f is not None)
        if ctx.want_params:
            saved.append(i_syn)
        ctx.save_for_backward(*saved)
        return spikes, v_mem, v_post_last, i_syn, i_last

    @staticmethod
    def backward(ctx, g_spikes, g_vmem, g_vlast, g_isyn, g_ilast):
        B, T, M = ctx.geometry
        N = B * M
        saved = list(ctx.saved_tensors)
        v_mem = saved.pop(0)
        f = {k: None for k in ("a_syn", "s_syn", "a_mem", "s_mem", "th", "c", "lo")}
        for k in ctx.keys:
            f[k] = saved.pop(0)
        vi_f = saved.pop(0) if ctx.has_init[0] else None
        ii_f = saved.pop(0) if ctx.has_init[1] else None
        i_syn = saved.pop(0) if ctx.want_params else None
        modes = ctx.modes
        dev = v_mem.device
        if g_spikes is None:
            g_spikes = torch.zeros_like(v_mem)
        g_spikes = g_spikes.contiguous()
        g_vmem = None if g_vmem is None else g_vmem.contiguous()
        g_isyn = None if g_isyn is None else g_isyn.contiguous()
        g_vlast = None if g_vlast is None else g_vlast.to(torch.float32).reshape(-1).contiguous()
        g_ilast = None if g_ilast is None else g_ilast.to(torch.float32).reshape(-1).contiguous()
        kind, p0, p1 = classify(ctx.surrogate_fn)
        surr = None
        if kind == _lib.SURR_GENERIC:
            th = f["th"]
            th_b = th if th.numel() == 1 else (th.view(1, 1, M) if modes["th"] == _lib.PARAM_PER_M else th.view(B, 1, M))
            surr = ctx.surrogate_fn(v_mem, th_b).to(torch.float32).contiguous()
        new = lambda: torch.empty(N, dtype=torch.float32, device=dev)
        grad_input = torch.empty_like(v_mem)
        gv0 = new() if ctx.init_shapes[0] is not None else None
        gi0 = new() if ctx.init_shapes[1] is not None else None
        spec = lambda k: (f[k], modes[k])
        tail = (gv0, gi0, g_spikes, g_vmem, g_vlast, g_isyn, g_ilast, v_mem, i_syn, surr, vi_f, ii_f, spec("a_syn"),
                spec("s_syn"), spec("s_mem"), spec("a_mem"), spec("c"), spec("th"), spec("lo"), ctx.max_spikes,
                ctx.reset_mode, kind, p0, p1, B, T, M)
        if gv0 is not None:
            gv0 = gv0.reshape(ctx.init_shapes[0])
        if gi0 is not None:
            gi0 = gi0.reshape(ctx.init_shapes[1])
        if ctx.acc is not None:
            # both decays' gradients reduced over the batch, with their scale parts and chain rules, in the kernel
            _lib.lif_syn_backward(grad_input, None, None, None, None, *tail, acc_decay_mem=ctx.acc[0], acc_decay_syn=ctx.acc[1])
            g_mem = torch.empty(f["a_mem"].numel(), dtype=torch.float32, device=dev)
            g_syn = torch.empty(f["a_syn"].numel(), dtype=torch.float32, device=dev)
            _lib.acc_finish(g_mem, ctx.acc[0])
            _lib.acc_finish(g_syn, ctx.acc[1])
            return (grad_input, g_syn.reshape(ctx.param_shapes["a_syn"]) if ctx.param_needs["a_syn"] else None, None, gi0,
                    g_mem.reshape(ctx.param_shapes["a_mem"]) if ctx.param_needs["a_mem"] else None, None, gv0,
                    None, None, None, None, None, None, None, None, None, None)
        ga_mem, gs_mem, ga_syn, gs_syn = (new(), new(), new(), new()) if ctx.want_params else (None,) * 4
        _lib.lif_syn_backward(grad_input, ga_mem, gs_mem, ga_syn, gs_syn, *tail)

        def red(per_instance, key):
            if not ctx.param_needs[key]:
                return None
            return _reduce_to_param(per_instance, ctx.param_shapes[key], modes[key] & _lib.PARAM_SHAPE_MASK, B, M)

        if any(ctx.flags):
            # derived decays / scales on a shape-independent route: fold with PyTorch what the kernel left per instance
            def fold(key_a, key_s, decay_flags, scale_flags, ga, gs):
                if not ctx.param_needs[key_a]:
                    return None
                shape, mode = ctx.param_shapes[key_a], modes[key_a] & _lib.PARAM_SHAPE_MASK
                g = _reduce_to_param(ga, shape, mode, B, M)
                gs_p = _reduce_to_param(gs, shape, mode, B, M) if scale_flags else None
                return _fold_decay_grad(g, gs_p, f[key_a].reshape(shape), decay_flags, scale_flags, None)
            fl = ctx.flags
            return (grad_input, fold("a_syn", "s_syn", fl[0], fl[1], ga_syn, gs_syn), None if fl[1] else red(gs_syn, "s_syn"),
                    gi0, fold("a_mem", "s_mem", fl[2], fl[3], ga_mem, gs_mem), None if fl[3] else red(gs_mem, "s_mem"),
                    gv0, None, None, None, None, None, None, None, None, None, None)

        return (grad_input, red(ga_syn, "a_syn"), red(gs_syn, "s_syn"), gi0, red(ga_mem, "a_mem"), red(gs_mem, "s_mem"),
                gv0, None, None, None, None, None, None, None, None, None, None)
