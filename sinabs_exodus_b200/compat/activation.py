"""Activation tokens and surrogate-gradient callables.

The exodus layers use the spike and reset objects only as tokens that carry
attributes (reference ``layers/lif.py:130-150``): the spike and reset
arithmetic itself runs inside the CUDA kernel.  The surrogate callables are
evaluated as ``fn(v_mem, spike_threshold)`` (reference ``spike.py:251``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import HAVE_SINABS

if HAVE_SINABS:  # pragma: no cover - depends on the environment
    from sinabs.activation import (  # type: ignore  # noqa: F401
        Heaviside,
        MaxSpike,
        MembraneReset,
        MembraneSubtract,
        MultiSpike,
        PeriodicExponential,
        SingleExponential,
        SingleSpike,
    )
else:

    class MultiSpike:
        """Token: a neuron may emit several spikes per step, floor(v / threshold)."""

    class SingleSpike:
        """Token: at most one spike per step."""

    @dataclass
    class MaxSpike:
        """At most ``max_num_spikes_per_bin`` spikes per step."""

        max_num_spikes_per_bin: Optional[int] = None

    @dataclass
    class MembraneSubtract:
        """After spiking, ``subtract_value`` (default: the threshold) is subtracted per spike."""

        subtract_value: Optional[float] = None

    @dataclass
    class MembraneReset:
        """After spiking, the membrane potential is set to ``reset_value``."""

        reset_value: float = 0.0

    @dataclass
    class SingleExponential:
        """s(v) = grad_scale / w * exp(-|v - theta| / w) with w = grad_width * theta."""

        grad_width: float = 0.5
        grad_scale: float = 1.0

        def __call__(self, v_mem: torch.Tensor, spike_threshold) -> torch.Tensor:
            width = spike_threshold * self.grad_width
            return self.grad_scale / width * torch.exp(-torch.abs(v_mem - spike_threshold) / width)

    @dataclass
    class Heaviside:
        """s(v) = 1/theta where v >= theta - window, else 0."""

        window: float = 1.0

        def __call__(self, v_mem: torch.Tensor, spike_threshold) -> torch.Tensor:
            return (v_mem >= (spike_threshold - self.window)).to(v_mem.dtype) / spike_threshold

    @dataclass
    class PeriodicExponential:
        """Exponential bump around the threshold, repeated with period theta above it.

        u = v - theta/2;  w = u below threshold, u - floor(u / theta) at or above it;
        s(v) = grad_scale * exp(-|w - theta/2| / grad_width) / theta.
        """

        grad_width: float = 0.5
        grad_scale: float = 1.0

        def __call__(self, v_mem: torch.Tensor, spike_threshold) -> torch.Tensor:
            half = spike_threshold / 2
            u = v_mem - half
            periodic = u - torch.floor(u / spike_threshold)
            w = torch.where(v_mem >= spike_threshold, periodic, u)
            return self.grad_scale * torch.exp(-torch.abs(w - half) / self.grad_width) / spike_threshold
