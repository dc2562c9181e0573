"""Whole-step CUDA-graph capture for networks built from the EXODUS layers.

For small problems a step is bound by launch and framework overhead, not by the kernels (a
``(8, 100, 128)`` LIF step: 0.05 ms of kernels inside 0.7 ms of host work).  The layers make no
host-device synchronisation in their steady state, so a step (state handling, forward and,
for training, backward) can be captured once and replayed with one launch.

``GraphedStep`` wraps the capture protocol of ``torch.cuda.CUDAGraph``: warm-up on a side
stream, static input / gradient buffers, gradients recreated inside the capture so that they
live in the graph's memory pool, and the layers' state buffers (``v_mem``, ``i_syn``), which
the layers *replace* on every call, turned into fixed tensors that the graph updates in place.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import nn

__all__ = ["GraphedStep"]


def _stateful_modules(module: nn.Module) -> List[nn.Module]:
    return [m for m in module.modules() if callable(getattr(m, "reset_states", None))]


class GraphedStep:
    """One forward (and backward) pass of ``module`` as a replayable CUDA graph.

    Parameters
    ----------
    module: the network; every stateful layer in it must be an EXODUS layer (or at least keep
        its state in buffers and expose ``reset_states``).
    example_input: CUDA tensor with the shape every call will use.
    example_grad: upstream gradient for ``module(example_input)``; given -> the step is
        ``zero_grad``, forward, ``backward(grad)``; ``None`` -> forward only, under ``no_grad``.
    carry_state: ``False`` resets the layers' states at the start of every step (independent
        samples).  ``True`` keeps them from one call to the next, detached (streaming inference,
        truncated BPTT): the state buffers become fixed tensors that each replay reads and then
        overwrites.
    input_grad: also produce the gradient w.r.t. the input (``.input_grad`` after a call).

    Calling the object copies ``x`` (and ``grad``) into the static buffers, replays the graph and
    returns the static output tensor, which the next call overwrites.  Parameter gradients are
    in ``param.grad`` as after an eager step; their tensors are those of the graph's memory pool
    and are refilled (not accumulated into) by every replay.

    What is captured is what ran during the capture: shapes, layer options and the set of
    parameters that require gradients are frozen; parameter *values* are read at replay time, so
    an optimizer that updates them in place works between replays.  Frozen too are the decisions the
    layers take from parameter values on the host: the value checks (0 <= alpha <= 1, threshold >
    min_v_mem) ran during the warm-up and are not repeated by a replay, and so did the choice of how
    the ``norm_input`` scale gradient is formed (rebuilt from the membrane potential while
    1 - alpha >= 0.01, from the input otherwise).  An optimizer that can move a time constant across
    those limits should re-capture.
    """

    def __init__(self, module: nn.Module, example_input: torch.Tensor, example_grad: Optional[torch.Tensor] = None,
                 *, carry_state: bool = False, input_grad: bool = False, warmup: int = 3):
        if not example_input.is_cuda:
            raise ValueError("GraphedStep needs CUDA tensors: the layers have no CPU implementation")
        self.module = module
        self.training_step = example_grad is not None
        self.carry_state = carry_state
        self._stateful = _stateful_modules(module)
        self.static_input = example_input.detach().clone()
        if self.training_step and input_grad:
            self.static_input.requires_grad_(True)
        self.static_grad = example_grad.detach().clone() if self.training_step else None
        self.static_output: Optional[torch.Tensor] = None
        self.input_grad: Optional[torch.Tensor] = None
        self._fixed_state: List[Tuple[nn.Module, str, torch.Tensor]] = []

        dev = example_input.device
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):     # first calls initialise states, run the value checks, size the pools
                self._step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)

        if carry_state:
            for m in self._stateful:
                for name, buf in list(m.named_buffers(recurse=False)):
                    fixed = buf.detach().clone()
                    m.register_buffer(name, fixed)
                    self._fixed_state.append((m, name, fixed))
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            out = self._step()
            for m, name, fixed in self._fixed_state:
                new = getattr(m, name)
                if new is not fixed:
                    fixed.copy_(new.detach())
                    m.register_buffer(name, fixed)
        self.static_output = out
        if self.training_step and input_grad:
            self.input_grad = self.static_input.grad
        torch.cuda.synchronize(dev)

    def _step(self) -> torch.Tensor:
        if not self.carry_state:
            for m in self._stateful:
                m.reset_states()
        elif self.training_step:
            # Truncated back-propagation: the states come from the previous step, whose graph is gone.  Cut them
            # here, layer by layer; `module.zero_grad()` below only reaches a layer's own override when `module`
            # is that layer (nn.Module.zero_grad walks parameters, not the children's methods).
            for m in self._stateful:
                for name, buf in list(m.named_buffers(recurse=False)):
                    if buf.requires_grad or buf.grad_fn is not None:
                        m.register_buffer(name, buf.detach())
        if not self.training_step:
            with torch.no_grad():
                return self.module(self.static_input)
        self.module.zero_grad(set_to_none=True)
        self.static_input.grad = None
        out = self.module(self.static_input)
        out.backward(self.static_grad)
        return out.detach()

    def __call__(self, x: torch.Tensor, grad: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x is not self.static_input:
            self.static_input.detach().copy_(x)
        if self.training_step and grad is not None and grad is not self.static_grad:
            self.static_grad.copy_(grad)
        self.graph.replay()
        return self.static_output

    def replay(self) -> torch.Tensor:
        """Replay on whatever the static buffers hold (``static_input`` / ``static_grad`` filled by the caller)."""
        self.graph.replay()
        return self.static_output
