"""The layers that are special cases of ``LIF``: ``IAF`` (no leak), ``ExpLeak`` (no spikes), and the
``*Squeeze`` form of each for 4D ``(batch*time, channel, height, width)`` input.

Same constructor arguments, defaults and ``_param_dict`` contents as the reference layers
(``sinabs/exodus/layers/iaf.py:13-112``, ``exp_leak.py:7-91``, ``lif.py:313-329``).  Each variant is a
fixed set of ``LIF`` arguments plus the list of constructor keys it does not have; the Squeeze
forms are produced by one class factory.
"""
from __future__ import annotations

import math
import weakref
from typing import Callable, Optional, Union

import torch

from ..compat.activation import MembraneSubtract, MultiSpike, SingleExponential
from ..compat.layers import SqueezeMixin
from .lif import LIF, _scalar_constant

__all__ = ["IAF", "IAFSqueeze", "ExpLeak", "ExpLeakSqueeze", "LIFSqueeze"]

Number = Union[float, torch.Tensor]


class _Variant(LIF):
    """``LIF`` with some constructor arguments pinned; ``_absent`` lists those keys."""

    _absent: tuple = ()

    @property
    def _param_dict(self) -> dict:
        kept = dict(super()._param_dict)
        for key in self._absent:
            kept.pop(key, None)
        return kept


class IAF(_Variant):
    """Integrate-and-fire: a ``LIF`` whose membrane does not leak (``alpha_mem`` = 1, no input normalisation)."""

    _absent = ("tau_mem", "train_alphas", "norm_input")

    def __init__(self, spike_threshold: Optional[Number] = 1.0, spike_fn: Callable = MultiSpike,
                 reset_fn: Callable = MembraneSubtract(), surrogate_grad_fn: Callable = SingleExponential(),
                 tau_syn: Optional[Number] = None, min_v_mem: Optional[Number] = None,
                 shape: Optional[torch.Size] = None, record_states: bool = False, decay_early: bool = True):
        pinned = dict(tau_mem=math.inf, norm_input=False)
        super().__init__(spike_threshold=spike_threshold, spike_fn=spike_fn, reset_fn=reset_fn,
                         surrogate_grad_fn=surrogate_grad_fn, tau_syn=tau_syn, min_v_mem=min_v_mem, shape=shape,
                         record_states=record_states, decay_early=decay_early, **pinned)
        self.tau_mem = None      # the layer has no membrane time constant (reference iaf.py:80-81)

    @property
    def alpha_mem_calculated(self) -> torch.Tensor:
        # a constant made on the device, once: a host-to-device copy would stall the launch queue
        return _scalar_constant(1.0, self.v_mem.device).reshape(())


class ExpLeak(_Variant):
    """Leaky integrator without spiking; ``decay_early`` and ``norm_input`` default to ``False`` as in the reference."""

    _absent = ("tau_syn", "spike_fn", "reset_fn", "surrogate_grad_fn", "spike_threshold")

    def __init__(self, tau_mem: Number, shape: Optional[torch.Size] = None, train_alphas: bool = False,
                 min_v_mem: Optional[float] = None, norm_input: bool = False, record_states: bool = False,
                 decay_early: bool = False):
        pinned = dict(tau_syn=None, spike_threshold=None, spike_fn=None, reset_fn=None, surrogate_grad_fn=None)
        super().__init__(tau_mem=tau_mem, shape=shape, train_alphas=train_alphas, min_v_mem=min_v_mem,
                         norm_input=norm_input, record_states=record_states, decay_early=decay_early, **pinned)


def _squeezed(base: type, name: str) -> type:
    """The 4D-input form of ``base``: ``(batch*time, ...)`` is viewed as ``(batch, time, ...)`` around the call."""

    def __init__(self, batch_size=None, num_timesteps=None, **kwargs):
        base.__init__(self, **kwargs)
        self.squeeze_init(batch_size, num_timesteps)

    def forward(self, input_data: torch.Tensor) -> torch.Tensor:
        out = self.squeeze_forward(input_data, lambda x: base.forward(self, x))
        if out.requires_grad:      # the tensor the caller holds is the flattened one: firing_rate differentiates through it
            self._rate_output = weakref.ref(out)
        return out

    def _param_dict(self) -> dict:
        return self.squeeze_param_dict(base._param_dict.fget(self))

    return type(name, (base, SqueezeMixin), {
        "__init__": __init__, "forward": forward, "_param_dict": property(_param_dict),
        "__doc__": f"``{base.__name__}`` for 4D input (batch*time, channel, height, width).",
        "__module__": __name__, "__qualname__": name,
    })


LIFSqueeze = _squeezed(LIF, "LIFSqueeze")
IAFSqueeze = _squeezed(IAF, "IAFSqueeze")
ExpLeakSqueeze = _squeezed(ExpLeak, "ExpLeakSqueeze")
