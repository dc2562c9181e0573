"""EXODUS ``IAF`` layer: ``LIF`` without leak (reference ``sinabs/exodus/layers/iaf.py:13-112``)."""
from __future__ import annotations

from typing import Callable, Optional, Union

import numpy as np
import torch

from ..compat.activation import MembraneSubtract, MultiSpike, SingleExponential
from ..compat.layers import SqueezeMixin
from .lif import LIF, _scalar_constant

__all__ = ["IAF", "IAFSqueeze"]


class IAF(LIF):
    """Integrate-and-fire layer; parameters as the reference layer (no ``tau_mem``, no ``norm_input``)."""

    def __init__(
        self,
        spike_threshold: Optional[Union[float, torch.Tensor]] = 1.0,
        spike_fn: Callable = MultiSpike,
        reset_fn: Callable = MembraneSubtract(),
        surrogate_grad_fn: Callable = SingleExponential(),
        tau_syn: Optional[Union[float, torch.Tensor]] = None,
        min_v_mem: Optional[Union[float, torch.Tensor]] = None,
        shape: Optional[torch.Size] = None,
        record_states: bool = False,
        decay_early: bool = True,
    ):
        super().__init__(
            tau_mem=np.inf,
            tau_syn=tau_syn,
            spike_threshold=spike_threshold,
            spike_fn=spike_fn,
            reset_fn=reset_fn,
            surrogate_grad_fn=surrogate_grad_fn,
            min_v_mem=min_v_mem,
            shape=shape,
            norm_input=False,
            record_states=record_states,
            decay_early=decay_early,
        )
        # IAF has no membrane time constant (reference iaf.py:80-81)
        self.tau_mem = None

    @property
    def alpha_mem_calculated(self):
        # made on the device, once (no host-to-device copy, which would stall the launch queue)
        return _scalar_constant(1.0, self.v_mem.device).reshape(())

    @property
    def _param_dict(self) -> dict:
        param_dict = super()._param_dict
        param_dict.pop("tau_mem")
        param_dict.pop("train_alphas")
        param_dict.pop("norm_input")
        return param_dict


class IAFSqueeze(IAF, SqueezeMixin):
    """``IAF`` for 4D input (batch*time, channel, height, width)."""

    def __init__(self, batch_size=None, num_timesteps=None, **kwargs):
        super().__init__(**kwargs)
        self.squeeze_init(batch_size, num_timesteps)

    def forward(self, input_data: torch.Tensor) -> torch.Tensor:
        return self.squeeze_forward(input_data, super().forward)

    @property
    def _param_dict(self) -> dict:
        return self.squeeze_param_dict(super()._param_dict)
