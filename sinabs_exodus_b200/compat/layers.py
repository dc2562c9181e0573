"""Base classes the exodus layers build on.

With ``sinabs`` installed these names are simply ``sinabs.layers.LIF``,
``IAF``, ``ExpLeak``, their ``Squeeze`` variants and ``SqueezeMixin``.  Without
it, the classes below provide the surface the reference layers rely on
(reference ``layers/lif.py:114-126,174-177,188,204,279``; tests
``tests/test_lif.py:23,63,222,477``): constructor arguments, the ``tau_mem`` /
``alpha_mem`` parameters, the ``v_mem`` / ``i_syn`` state buffers and their
helpers, ``_param_dict`` / ``arg_dict`` and ``__repr__``.

These stand-ins hold state and parameters only.  They have NO forward pass of
their own: this package computes on the GPU through its CUDA library and has
no PyTorch or CPU implementation of the neuron dynamics.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple, Union

import numpy as np
import torch
from torch import nn

from . import HAVE_SINABS
from .activation import MembraneSubtract, MultiSpike, SingleExponential

if HAVE_SINABS:  # pragma: no cover - depends on the environment
    from sinabs.layers import (  # type: ignore  # noqa: F401
        IAF,
        LIF,
        ExpLeak,
        ExpLeakSqueeze,
        IAFSqueeze,
        LIFSqueeze,
        SqueezeMixin,
    )
else:

    def _as_tensor(x) -> torch.Tensor:
        return x.detach().clone().float() if isinstance(x, torch.Tensor) else torch.as_tensor(x, dtype=torch.float32)

    class LIF(nn.Module):
        """State and parameter holder of a leaky integrate-and-fire layer."""

        def __init__(
            self,
            tau_mem: Union[float, torch.Tensor],
            tau_syn: Optional[Union[float, torch.Tensor]] = None,
            spike_threshold: Optional[Union[float, torch.Tensor]] = 1.0,
            spike_fn: Optional[Callable] = MultiSpike,
            reset_fn: Optional[Callable] = MembraneSubtract(),
            surrogate_grad_fn: Optional[Callable] = SingleExponential(),
            min_v_mem: Optional[Union[float, torch.Tensor]] = None,
            train_alphas: bool = False,
            shape: Optional[torch.Size] = None,
            norm_input: bool = True,
            record_states: bool = False,
        ):
            super().__init__()
            self.train_alphas = train_alphas
            tau_mem_t = _as_tensor(tau_mem)
            if train_alphas:
                self.alpha_mem = nn.Parameter(torch.exp(-1.0 / tau_mem_t))
                self.alpha_syn = nn.Parameter(torch.exp(-1.0 / _as_tensor(tau_syn))) if tau_syn is not None else None
            else:
                self.tau_mem = nn.Parameter(tau_mem_t)
                self.tau_syn = nn.Parameter(_as_tensor(tau_syn)) if tau_syn is not None else None
            self.spike_threshold = spike_threshold
            self.spike_fn = spike_fn
            self.reset_fn = reset_fn
            self.surrogate_grad_fn = surrogate_grad_fn
            self.min_v_mem = min_v_mem
            self.norm_input = norm_input
            self.record_states = record_states
            self.register_buffer("v_mem", torch.zeros(0))
            if tau_syn is not None:
                self.register_buffer("i_syn", torch.zeros(0))
            if shape is not None:
                self.init_state_with_shape(tuple(shape))
            self.recordings = dict()

        # -- time constants ---------------------------------------------------
        @property
        def alpha_mem_calculated(self) -> torch.Tensor:
            return self.alpha_mem if self.train_alphas else torch.exp(-1.0 / self.tau_mem)

        @property
        def alpha_syn_calculated(self) -> Optional[torch.Tensor]:
            if self.train_alphas:
                return self.alpha_syn
            return None if self.tau_syn is None else torch.exp(-1.0 / self.tau_syn)

        @property
        def tau_mem_calculated(self) -> torch.Tensor:
            return -1.0 / torch.log(self.alpha_mem) if self.train_alphas else self.tau_mem

        @property
        def tau_syn_calculated(self) -> Optional[torch.Tensor]:
            if self.train_alphas:
                return None if self.alpha_syn is None else -1.0 / torch.log(self.alpha_syn)
            return self.tau_syn

        # -- state ------------------------------------------------------------
        @property
        def does_spike(self) -> bool:
            return self.spike_fn is not None

        def is_state_initialised(self) -> bool:
            return all(b.numel() > 0 for b in self.buffers())

        def state_has_shape(self, shape: Tuple[int, ...]) -> bool:
            return all(tuple(b.shape) == tuple(shape) for b in self.buffers())

        def init_state_with_shape(self, shape: Tuple[int, ...], randomize: bool = False) -> None:
            for name, buf in list(self.named_buffers()):
                new = torch.rand(shape, device=buf.device) if randomize else torch.zeros(shape, device=buf.device)
                self.register_buffer(name, new)

        def reset_states(self, randomize: bool = False, value_ranges=None) -> None:
            if not self.is_state_initialised():
                return
            for name, buf in list(self.named_buffers()):
                new = torch.rand_like(buf.detach()) if randomize else torch.zeros_like(buf.detach())
                if randomize and value_ranges and name in value_ranges:
                    lo, hi = value_ranges[name]
                    new = new * (hi - lo) + lo
                self.register_buffer(name, new)

        def zero_grad(self, set_to_none: bool = True) -> None:
            # Cut the graph that the states carry from one forward call to the next.
            bufs = self._buffers      # the layer has no submodules
            for name, buf in bufs.items():
                if buf is not None and (buf.grad_fn is not None or buf.requires_grad):
                    bufs[name] = buf.detach()
            super().zero_grad(set_to_none)

        # -- construction arguments -------------------------------------------
        @property
        def _param_dict(self) -> dict:
            tau_mem = self.tau_mem_calculated
            tau_syn = self.tau_syn_calculated
            return dict(
                tau_mem=None if tau_mem is None else tau_mem.detach(),
                tau_syn=None if tau_syn is None else tau_syn.detach(),
                spike_threshold=self.spike_threshold,
                spike_fn=self.spike_fn,
                reset_fn=self.reset_fn,
                surrogate_grad_fn=self.surrogate_grad_fn,
                min_v_mem=self.min_v_mem,
                train_alphas=self.train_alphas,
                shape=tuple(self.v_mem.shape) if self.v_mem.numel() else None,
                norm_input=self.norm_input,
                record_states=self.record_states,
            )

        @property
        def arg_dict(self) -> dict:
            return dict(self._param_dict)

        def forward(self, input_data: torch.Tensor):  # pragma: no cover - deliberate
            raise NotImplementedError(
                "This stand-in for sinabs.layers.LIF holds parameters and state only. "
                "Use the EXODUS layers (CUDA) or install sinabs for its PyTorch layers.")

        def __repr__(self) -> str:
            args = ", ".join(f"{k}={v}" for k, v in self._param_dict.items()
                             if k in ("tau_mem", "tau_syn", "spike_threshold", "min_v_mem", "train_alphas"))
            return f"{type(self).__name__}({args}, batch_size={self.v_mem.shape[0] if self.v_mem.numel() else None})"

    class IAF(LIF):
        """Integrate-and-fire: LIF without leak."""

        def __init__(self, spike_threshold=1.0, spike_fn=MultiSpike, reset_fn=MembraneSubtract(),
                     surrogate_grad_fn=SingleExponential(), tau_syn=None, min_v_mem=None, shape=None,
                     record_states=False):
            super().__init__(tau_mem=np.inf, tau_syn=tau_syn, spike_threshold=spike_threshold, spike_fn=spike_fn,
                             reset_fn=reset_fn, surrogate_grad_fn=surrogate_grad_fn, min_v_mem=min_v_mem,
                             shape=shape, norm_input=False, record_states=record_states)
            self.tau_mem = None

        @property
        def alpha_mem_calculated(self):
            return torch.tensor(1.0, device=self.v_mem.device)

        @property
        def _param_dict(self) -> dict:
            d = super()._param_dict
            for k in ("tau_mem", "train_alphas", "norm_input"):
                d.pop(k)
            return d

    class ExpLeak(LIF):
        """Leaky integrator without spiking."""

        def __init__(self, tau_mem, shape=None, train_alphas=False, min_v_mem=None, norm_input=False,
                     record_states=False):
            super().__init__(tau_mem=tau_mem, tau_syn=None, spike_threshold=None, train_alphas=train_alphas,
                             min_v_mem=min_v_mem, shape=shape, spike_fn=None, reset_fn=None,
                             surrogate_grad_fn=None, norm_input=norm_input, record_states=record_states)

        @property
        def _param_dict(self) -> dict:
            d = super()._param_dict
            for k in ("tau_syn", "spike_fn", "reset_fn", "surrogate_grad_fn", "spike_threshold"):
                d.pop(k)
            return d

    class SqueezeMixin:
        """Lets a layer take (batch*time, ...) input by unfolding it to (batch, time, ...)."""

        def squeeze_init(self, batch_size: Optional[int], num_timesteps: Optional[int]) -> None:
            if not batch_size and not num_timesteps:
                raise TypeError("You need to specify either batch_size or num_timesteps.")
            self.batch_size = batch_size if batch_size else -1
            self.num_timesteps = num_timesteps if num_timesteps else -1

        def squeeze_forward(self, input_data: torch.Tensor, forward_method: Callable) -> torch.Tensor:
            inflated = input_data.reshape(self.batch_size, self.num_timesteps, *input_data.shape[1:])
            return forward_method(inflated).flatten(start_dim=0, end_dim=1)

        def squeeze_param_dict(self, param_dict: dict) -> dict:
            param_dict.update(batch_size=self.batch_size, num_timesteps=self.num_timesteps)
            return param_dict

    class _SqueezeBase(SqueezeMixin):
        def __init__(self, batch_size=None, num_timesteps=None, **kwargs):
            super().__init__(**kwargs)
            self.squeeze_init(batch_size, num_timesteps)

        @property
        def _param_dict(self) -> dict:
            return self.squeeze_param_dict(super()._param_dict)

    class LIFSqueeze(_SqueezeBase, LIF):
        pass

    class IAFSqueeze(_SqueezeBase, IAF):
        pass

    class ExpLeakSqueeze(_SqueezeBase, ExpLeak):
        pass


def replace_module(model: nn.Module, source_class: type, mapper_fn: Callable) -> nn.Module:
    """Return ``model`` with every sub-module whose class is exactly ``source_class`` replaced by ``mapper_fn(module)``.

    Same contract as the helper the reference's conversion functions call
    (``conversion.py:35,59``); uses the sinabs implementation when available.
    """
    if HAVE_SINABS:  # pragma: no cover - depends on the environment
        import sinabs.conversion
        return sinabs.conversion.replace_module(model, source_class, mapper_fn=mapper_fn)
    if type(model) is source_class:
        return mapper_fn(model)
    for name, child in list(model.named_children()):
        setattr(model, name, replace_module(child, source_class, mapper_fn))
    return model
