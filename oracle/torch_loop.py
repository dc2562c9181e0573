"""Time-stepped pure-PyTorch neuron loop with autograd (test infrastructure, never shipped).

One Python iteration per time step, spike non-linearity as an autograd Function
whose backward multiplies by the surrogate gradient: back-propagation through
time over this loop is the ground truth the single-pass EXODUS backward is
equivalent to (Gradient_analysis.ipynb, cells 0 and 7 of the reference).  It is

* the checker for options the reference has no kernel for (reset to a value),
* the checker for the layer glue (layers/lif.py:152-307 of the reference:
  synaptic stage, decay_early, norm_input, state carry-over),
* the "time-stepped PyTorch layer on host cores" CPU baseline of the benchmark
  (the package the reference compares itself with is not installed here).

Layout is the layer's own: (batch, time, *neurons).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


class _Spike(torch.autograd.Function):
    """a = min(trunc(v / theta), max_spikes) where v >= theta, else 0;  da/dv := surrogate(v, theta)."""

    @staticmethod
    def forward(ctx, v, theta, surrogate_fn, max_spikes):
        ctx.save_for_backward(v, theta)
        ctx.surrogate_fn = surrogate_fn
        n = torch.where(v >= theta, torch.div(v, theta).trunc(), torch.zeros_like(v))
        if max_spikes is not None:
            n = torch.clamp(n, max=float(max_spikes))
        return n

    @staticmethod
    def backward(ctx, grad):
        v, theta = ctx.saved_tensors
        return grad * ctx.surrogate_fn(v, theta), None, None, None


def lif_loop(
    x: torch.Tensor,
    alpha_mem: torch.Tensor,
    v_init: torch.Tensor,
    theta: Optional[torch.Tensor] = None,
    subtract: Optional[torch.Tensor] = None,
    min_v_mem: Optional[torch.Tensor] = None,
    surrogate_fn: Optional[Callable] = None,
    max_spikes: Optional[int] = None,
    reset_value: Optional[float] = None,
    alpha_syn: Optional[torch.Tensor] = None,
    i_syn_init: Optional[torch.Tensor] = None,
    norm_input: bool = False,
    decay_early: bool = True,
    spiking: bool = True,
):
    """Evolve (B, T, *) input.  Returns dict(spikes, v_mem_pre, v_mem_post, i_syn, v_last, i_last).

    ``v_init`` is the state after the previous reset.  With ``spiking=False`` the
    membrane is a plain leaky integrator (the ExpLeak branch, layers/lif.py:211-223),
    where ``decay_early`` scales the input by alpha_mem.  ``reset_value`` not None
    selects "reset to a value where a spike occurred" instead of "subtract".
    """
    B, T = x.shape[:2]
    v = v_init
    i_syn = i_syn_init
    spikes, v_pre, v_post, i_all = [], [], [], []
    for t in range(T):
        cur = x[:, t]
        if alpha_syn is not None:                      # layers/lif.py:185-198
            if decay_early:
                cur = cur * alpha_syn
            i_syn = alpha_syn * i_syn + cur
            cur = i_syn
            i_all.append(i_syn)
        if norm_input:                                 # layers/lif.py:206-209
            cur = (1.0 - alpha_mem) * cur
        if not spiking:
            if decay_early:                            # layers/lif.py:213-214
                cur = cur * alpha_mem
            v = alpha_mem * v + cur
            v_pre.append(v); v_post.append(v)
            continue
        v = alpha_mem * v + cur
        if min_v_mem is not None:                      # gradient 0 where clipped (strict >)
            v = torch.where(v > min_v_mem, v, min_v_mem.expand_as(v).detach())
        a = _Spike.apply(v, theta.expand_as(v), surrogate_fn, max_spikes)
        v_pre.append(v)
        spikes.append(a)
        if reset_value is None:
            v = v - subtract * a
        else:
            v = torch.where(a > 0, torch.full_like(v, reset_value), v)
        v_post.append(v)
    stack = lambda lst: torch.stack(lst, dim=1) if lst else None
    return dict(
        spikes=stack(spikes), v_mem_pre=stack(v_pre), v_mem_post=stack(v_post), i_syn=stack(i_all),
        v_last=v, i_last=i_syn,
    )
