"""EXODUS ``ExpLeak`` layer: non-spiking leaky integrator (reference ``sinabs/exodus/layers/exp_leak.py:7-91``)."""
from __future__ import annotations

from typing import Optional, Union

import torch

from ..compat.layers import SqueezeMixin
from .lif import LIF

__all__ = ["ExpLeak", "ExpLeakSqueeze"]


class ExpLeak(LIF):
    """Leaky integrator layer; ``decay_early`` and ``norm_input`` default to ``False`` as in the reference."""

    def __init__(
        self,
        tau_mem: Union[float, torch.Tensor],
        shape: Optional[torch.Size] = None,
        train_alphas: bool = False,
        min_v_mem: Optional[float] = None,
        norm_input: bool = False,
        record_states: bool = False,
        decay_early: bool = False,
    ):
        super().__init__(
            tau_mem=tau_mem,
            tau_syn=None,
            spike_threshold=None,
            train_alphas=train_alphas,
            min_v_mem=min_v_mem,
            shape=shape,
            spike_fn=None,
            reset_fn=None,
            surrogate_grad_fn=None,
            norm_input=norm_input,
            record_states=record_states,
            decay_early=decay_early,
        )

    @property
    def _param_dict(self) -> dict:
        param_dict = super()._param_dict
        for key in ("tau_syn", "spike_fn", "reset_fn", "surrogate_grad_fn", "spike_threshold"):
            param_dict.pop(key)
        return param_dict


class ExpLeakSqueeze(ExpLeak, SqueezeMixin):
    """``ExpLeak`` for 4D input (batch*time, channel, height, width)."""

    def __init__(self, batch_size=None, num_timesteps=None, **kwargs):
        super().__init__(**kwargs)
        self.squeeze_init(batch_size, num_timesteps)

    def forward(self, input_data: torch.Tensor) -> torch.Tensor:
        return self.squeeze_forward(input_data, super().forward)

    @property
    def _param_dict(self) -> dict:
        return self.squeeze_param_dict(super()._param_dict)
