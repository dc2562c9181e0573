"""EXODUS ``LIF`` layer on the B200 kernels.

Same constructor, state handling, recordings, ``firing_rate`` and ``repr`` as the
reference layer (``sinabs/exodus/layers/lif.py:47-329``).  What differs is how the
work reaches the GPU: the layer's own ``(batch, time, *neurons)`` tensor is used
as it is (time-major), parameters are passed un-expanded, and the ``decay_early``
/ ``norm_input`` multiplications, the state after the last reset and the spike
count are produced by the same kernel launch.  The reference's transpose copy
(``lif.py:181``), parameter broadcasts (``:188,204,226-243``), ``v - c*spikes``
pass (``:256``) and ``sum()/numel()`` pass (``:305``) have no counterpart here.
"""
from __future__ import annotations

import os
import weakref
from typing import Callable, Optional, Tuple, Union

import torch

from .. import _lib
from ..compat.activation import (
    MaxSpike,
    MembraneReset,
    MembraneSubtract,
    MultiSpike,
    SingleExponential,
    SingleSpike,
)
from ..compat.layers import LIF as LIFBase
from ..leaky import LeakyIntegratorTM
from ..spike import IntegrateAndFireTM, LIFSynapticTM, _flat32, _mode_of, acc_eligible, fused_synaptic_eligible

__all__ = ["LIF"]


def expand_to_1d_contiguous(value: Union[float, torch.Tensor], shape: Tuple[int]) -> torch.Tensor:
    """Expand ``value`` to ``shape``, flatten, make contiguous (reference ``lif.py:20-44``).

    Kept for API compatibility; the layers themselves never expand parameters.
    """
    return torch.as_tensor(value).expand(shape).float().flatten().contiguous()


_SCALARS: dict = {}


def _scalar_constant(value: float, device) -> torch.Tensor:
    """One-element tensor holding a Python number, made once per value and device (read-only).

    A fill kernel instead of a host-to-device copy: the copy would wait for all queued work.  Tensors
    made while a CUDA graph is being captured belong to that graph's memory pool and are not kept.
    """
    key = (value, str(device))
    t = _SCALARS.get(key)
    if t is None:
        t = torch.full((1,), value, dtype=torch.float32, device=device)
        if t.device.type != "cuda" or not torch.cuda.is_current_stream_capturing():
            _SCALARS[key] = t
    return t


def _flat_param(value, trailing: Tuple[int, ...], batch: int, device, perm=None) -> Optional[torch.Tensor]:
    """Bring a parameter to 1, M or B*M elements without breaking its autograd graph.

    A value that broadcasts against the neuron dimensions becomes M elements, one
    that needs the batch dimension too becomes B*M, a single value stays single.
    ``perm``: order in which the neuron dimensions lie in the input's memory (None = as given); the
    flattened parameter follows the same order.
    """
    if value is None:
        return None
    if isinstance(value, (int, float)):
        return _scalar_constant(float(value), device)
    t = value if isinstance(value, torch.Tensor) else torch.as_tensor(value, dtype=torch.float32)
    if t.device != torch.device(device) or t.dtype != torch.float32:
        t = t.to(device=device, dtype=torch.float32)
    if t.numel() == 1:
        return t.reshape(1)
    try:
        t = t.expand(trailing)
        lead = 0
    except RuntimeError:
        t = t.expand((batch, *trailing))
        lead = 1
    if perm is not None:
        t = t.permute(*range(lead), *[lead + d for d in perm])
    return t.reshape(-1)


class _DecayFromTau(torch.autograd.Function):
    """``alpha = exp(-1/tau)`` and, on request, ``1 - alpha`` (the ``norm_input`` scale) as ONE autograd node.

    Same values as the expression the layers are specified with (``torch.exp(-1.0 / tau)``); written as a
    Function because the four small nodes it replaces, and their four backward nodes, cost more host time per
    step than the neuron kernels of a small layer take to run.
    """

    @staticmethod
    def forward(ctx, tau, with_complement: bool):
        r = torch.reciprocal(tau)
        alpha = torch.exp(r.neg())
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(alpha, r)
        if with_complement:
            return alpha, 1.0 - alpha
        return alpha, None

    @staticmethod
    def backward(ctx, grad_alpha, grad_complement):
        alpha, r = ctx.saved_tensors
        if grad_alpha is None and grad_complement is None:
            return None, None
        if grad_complement is None:
            g = grad_alpha
        elif grad_alpha is None:
            g = grad_complement.neg()
        else:
            g = grad_alpha - grad_complement
        return g * alpha * r * r, None      # d/dtau exp(-1/tau) = exp(-1/tau) / tau^2


_SM_COUNT: dict = {}      # device -> number of SMs


class LIF(LIFBase):
    """Leaky integrate-and-fire layer, forward and exact backward on the GPU.

    Parameters are those of the reference layer: ``tau_mem``, ``tau_syn``,
    ``spike_threshold``, ``spike_fn`` (``MultiSpike``, ``SingleSpike`` or
    ``MaxSpike(k)``; ``None`` for a non-spiking integrator), ``reset_fn``,
    ``surrogate_grad_fn``, ``min_v_mem``, ``train_alphas``, ``shape``,
    ``norm_input``, ``record_states`` and ``decay_early``.

    Beyond the reference, ``reset_fn`` may be ``MembraneReset(value)``: the
    membrane is then set to ``value`` wherever a spike occurred, and the reset is
    treated as a constant mask in the backward pass.
    """

    def __init__(
        self,
        tau_mem: Union[float, torch.Tensor],
        tau_syn: Optional[Union[float, torch.Tensor]] = None,
        spike_threshold: Optional[Union[float, torch.Tensor]] = 1.0,
        spike_fn: Callable = MultiSpike,
        reset_fn: Callable = MembraneSubtract(),
        surrogate_grad_fn: Callable = SingleExponential(),
        min_v_mem: Optional[Union[float, torch.Tensor]] = None,
        train_alphas: bool = False,
        shape: Optional[torch.Size] = None,
        norm_input: bool = True,
        record_states: bool = False,
        decay_early: bool = True,
    ):
        self._parse_activation_fn(spike_fn, reset_fn)
        super().__init__(
            tau_mem=tau_mem,
            tau_syn=tau_syn,
            spike_threshold=spike_threshold,
            spike_fn=spike_fn,
            reset_fn=reset_fn,
            surrogate_grad_fn=surrogate_grad_fn,
            min_v_mem=min_v_mem,
            train_alphas=train_alphas,
            shape=shape,
            norm_input=norm_input,
            record_states=record_states,
        )
        self.decay_early = decay_early

    # 0: off; 1: where it pays; 2: wherever the kernels take the shape.  Default from the environment.
    _recompute = {"1": 1, "always": 2}.get(os.environ.get("EXODUS_B200_BACKWARD_RECOMPUTE", "0"), 0)

    def set_backward_recompute(self, enabled: bool = True, always: bool = False) -> None:
        """Training without the membrane-potential tensor.  The reference's forward writes ``v_mem`` for every
        neuron and step and its backward reads it back (``sinabs/exodus/spike.py:200,246``); a layer that does not
        record states needs it for nothing else.  With this switch on, the forward kernel writes the spikes and one
        checkpoint of the state per 8 steps, and the backward kernel rebuilds ``v_mem`` chunk by chunk from the
        layer's input and the checkpoints with the forward kernel's own arithmetic -- bit for bit the same tensor,
        hence the same gradients -- at 21 instead of 24 bytes per neuron and step and without 7/8 of ``v_mem``'s
        memory.  Applies to spiking layers without a synaptic stage (or in front of it: the membrane stage of the
        two-kernel route), built-in surrogate gradients, shapes the TMA-staged kernels take; anything else runs as
        before.

        The rebuild costs instructions, which only a problem that keeps the memory system busy can hide: measured
        +7 to +12 % on 32 x 500 x 262144 and +8 % on 32 x 300 x 36992, nothing on 64 x 500 x 4096, and -14 to -26 % on
        32 x 300 x 2048 and 16 x 1000 x 1024.  So by default it is used only when the batch gives at least eight
        512-neuron tiles per SM; ``always=True`` uses it for every shape the kernels take (for its memory saving).
        ``EXODUS_B200_BACKWARD_RECOMPUTE=1`` (or ``always``) in the environment turns it on for every layer."""
        self.__dict__["_recompute"] = (2 if always else 1) if enabled else 0

    def _recompute_here(self, x: torch.Tensor) -> bool:
        """Whether this (B, T, M) input takes the route without v_mem (see set_backward_recompute)."""
        if self._recompute == 2:
            return True
        if self._recompute == 0:
            return False
        sms = _SM_COUNT.get(x.device)
        if sms is None:
            sms = _SM_COUNT[x.device] = torch.cuda.get_device_properties(x.device).multi_processor_count
        return x.shape[0] * ((x.shape[2] + 511) // 512) >= 8 * sms

    def _set_state(self, name: str, value: torch.Tensor) -> None:
        # what ``self.<name> = value`` does for a registered buffer, without nn.Module.__setattr__'s searches
        self._buffers[name] = value

    def reset_states(self, randomize: bool = False, value_ranges=None) -> None:
        """Reset the states to zero (or, with ``randomize``, as the base class does).

        A plain reset installs a zero tensor that the layer keeps for this purpose instead of filling a new one on
        every call (one launch less per step for loops that reset between samples).  The forward pass never writes
        into its initial state, so the tensor stays zero; should anybody have modified it in place since it was
        installed (its version counter tells), a fresh one is made.
        """
        if randomize or not self.is_state_initialised():
            return super().reset_states(randomize=randomize, value_ranges=value_ranges)
        cache = self.__dict__.setdefault("_zero_states", {})
        bufs = self._buffers
        for name, buf in bufs.items():
            hit = cache.get(name)
            if hit is None or hit[0].shape != buf.shape or hit[0].device != buf.device or hit[0]._version != hit[1] \
                    or (hit[0].is_cuda and torch.cuda.is_current_stream_capturing()):
                z = torch.zeros_like(buf.detach())
                if not (z.is_cuda and torch.cuda.is_current_stream_capturing()):
                    cache[name] = (z, z._version)
            else:
                z = hit[0]
            bufs[name] = z

    def _parse_activation_fn(self, spike_fn, reset_fn):
        if spike_fn is None:
            return
        spike_ok = spike_fn in (MultiSpike, SingleSpike) or isinstance(spike_fn, MaxSpike)
        reset_ok = isinstance(reset_fn, (MembraneSubtract, MembraneReset))
        if not spike_ok or not reset_ok:
            raise NotImplementedError(
                "Spike mechanism config not supported. "
                "Use MultiSpike/SingleSpike/MaxSpike and MembraneSubtract (or MembraneReset) functions.")
        if isinstance(spike_fn, MaxSpike):
            self.max_num_spikes_per_bin = spike_fn.max_num_spikes_per_bin
        elif spike_fn == MultiSpike:
            self.max_num_spikes_per_bin = None
        else:
            self.max_num_spikes_per_bin = 1

    # ------------------------------------------------------------------
    def _prepare_input(self, input_data: torch.Tensor):
        """Initialise states if needed and view the input as (B, T, M)."""
        batch_size, time_steps, *trailing_dim = input_data.shape
        if not self.is_state_initialised() or not self.state_has_shape((batch_size, *trailing_dim)):
            self.init_state_with_shape((batch_size, *trailing_dim))
        x = input_data
        if x.dtype != torch.float32:
            x = x.float()
        neurons = 1
        for d in trailing_dim:
            neurons *= d
        # Neurons are independent, so the order in which they lie in memory is as good as any: an input whose
        # neuron dimensions are stored in another order (a `channels_last` feature map from a convolution in front
        # of a Squeeze layer, say) is used where it lies, with parameters, states and outputs following that order,
        # instead of being copied into the row-major order first.
        self._perm = None
        if len(trailing_dim) > 1 and not x.is_contiguous():
            order = sorted(range(len(trailing_dim)), key=lambda d: (-x.stride(2 + d), d))
            if order != list(range(len(trailing_dim))):
                xp = x.permute(0, 1, *[2 + d for d in order])
                if xp.is_contiguous():
                    self._perm = tuple(order)
                    x = xp
        x = x.reshape(batch_size, time_steps, neurons)
        if not x.is_contiguous():
            x = x.contiguous()
        return x, (batch_size, time_steps, *trailing_dim)

    def _membrane_decay(self):
        """(alpha_mem, 1 - alpha_mem or None): the decay per step and the ``norm_input`` scale."""
        tau = None if self.train_alphas else getattr(self, "tau_mem", None)
        if isinstance(tau, torch.Tensor):
            return _DecayFromTau.apply(tau, bool(self.norm_input))
        alpha = self.alpha_mem_calculated
        return alpha, ((1.0 - alpha) if self.norm_input else None)

    def _synaptic_decay(self):
        tau = None if self.train_alphas else getattr(self, "tau_syn", None)
        if isinstance(tau, torch.Tensor):
            return _DecayFromTau.apply(tau, False)[0]
        return self.alpha_syn_calculated

    _perm = None      # order of the neuron dimensions in the current input's memory (None: as declared)

    def _state_flat(self, state: torch.Tensor) -> torch.Tensor:
        """A (batch, *neurons) state as the flat vector the kernels index, neurons in the input's memory order."""
        if self._perm is not None and state.dim() == 1 + len(self._perm):
            state = state.permute(0, *[1 + d for d in self._perm])
        return state.reshape(-1)

    def _unflatten(self, t: torch.Tensor, lead: Tuple[int, ...], trailing: Tuple[int, ...]) -> torch.Tensor:
        """(*lead, M) in the kernels' neuron order -> (*lead, *trailing) in the declared order; a view either way, so an
        output computed on a `channels_last` input comes back in `channels_last` memory."""
        if self._perm is None:
            return t.reshape(*lead, *trailing)
        t = t.reshape(*lead, *[trailing[d] for d in self._perm])
        inverse = sorted(range(len(self._perm)), key=lambda i: self._perm[i])
        return t.permute(*range(len(lead)), *[len(lead) + i for i in inverse])

    def _decay_source(self, which: str):
        """``(tensor, flags)`` for the decay of the membrane (``"mem"``) or synapse (``"syn"``) stage: what the layer
        owns -- the time constant (``PARAM_IS_TAU``: the kernels form ``exp(-1/tau)`` themselves, and their backward
        returns the gradient w.r.t. tau) or, with ``train_alphas`` or a layer without leak, alpha itself."""
        if not self.train_alphas:
            tau = getattr(self, "tau_" + which, None)
            if isinstance(tau, torch.Tensor):
                return tau, _lib.PARAM_IS_TAU
        return getattr(self, f"alpha_{which}_calculated"), 0

    @staticmethod
    def _aux(n_acc: int, dev) -> torch.Tensor:
        """One zeroed float64 buffer per call: element 0 is the forward kernel's total (spike count, read as int64,
        or the output sum), the rest are the accumulators the backward kernel reduces parameter gradients into."""
        return torch.zeros(1 + n_acc, dtype=torch.float64, device=dev)

    def _forward_synaptic(self, x: torch.Tensor, batch: int, trailing):
        raw, dflags = self._decay_source("syn")
        raw = _flat_param(raw, trailing, batch, x.device, self._perm)
        acc = None
        if raw.requires_grad and torch.is_grad_enabled() and acc_eligible(x):
            acc = torch.zeros(raw.numel(), dtype=torch.float64, device=x.device)
        return LeakyIntegratorTM.apply(x, raw, self._state_flat(self.i_syn), None, None, dflags,
                                       _lib.SCALE_TIMES_ALPHA if self.decay_early else 0, acc)

    def _forward_membrane(self, i_syn: torch.Tensor, batch: int, trailing):
        dev = i_syn.device
        raw, dflags = self._decay_source("mem")
        raw = _flat_param(raw, trailing, batch, dev, self._perm)
        sflags = _lib.SCALE_ONE_MINUS_ALPHA if self.norm_input else 0
        use_acc = raw.requires_grad and torch.is_grad_enabled() and acc_eligible(i_syn)
        aux = self._aux(raw.numel() if use_acc else 0, dev)
        acc = aux[1:] if use_acc else None

        if self.spike_fn is None:
            if self.decay_early:
                sflags |= _lib.SCALE_TIMES_ALPHA
            total = aux[:1]
            v_mem, v_last = LeakyIntegratorTM.apply(i_syn, raw, self._state_flat(self.v_mem), None, total, dflags, sflags, acc)
            return v_mem, v_mem, v_last, total

        threshold = _flat_param(self.spike_threshold, trailing, batch, dev, self._perm)
        min_v_mem = _flat_param(self.min_v_mem, trailing, batch, dev, self._perm)
        if isinstance(self.reset_fn, MembraneReset):
            reset_mode = _lib.RESET_TO_VALUE
            subtract = _flat_param(self.reset_fn.reset_value, trailing, batch, dev, self._perm)
        else:
            reset_mode = _lib.RESET_SUBTRACT
            subtract = _flat_param(self.reset_fn.subtract_value, trailing, batch, dev, self._perm)
        self._validate_once(dev)
        count = aux[:1].view(torch.int64)
        # With autograd off the recorded potential is a plain side output of the forward launch; with autograd on
        # it stays the reference's differentiable expression (layers/lif.py:256), so that a loss on a recording works.
        fused_record = self.record_states and not torch.is_grad_enabled()
        v_rec = torch.empty_like(i_syn) if fused_record else None
        scale_from_state = bool(sflags) and getattr(self, "_scale_nonzero", False)
        # v_mem is an intermediate unless it is recorded: with set_backward_recompute the kernels keep checkpoints
        # instead (a derived scale's gradient is then rebuilt from the state, which needs the scale away from zero)
        recompute = (self._recompute and not self.record_states and torch.is_grad_enabled()
                     and (not sflags or scale_from_state) and self._recompute_here(i_syn))
        spikes, v_pre, v_post_last = IntegrateAndFireTM.apply(
            i_syn, raw, self._state_flat(self.v_mem), threshold, subtract, min_v_mem, None,
            self.surrogate_grad_fn, self.max_num_spikes_per_bin, reset_mode, count,
            scale_from_state, v_rec, dflags, sflags, acc, recompute,
            torch.is_grad_enabled() or self.record_states)      # inference without recording: spikes only
        if self.record_states and not fused_record:
            c = threshold if subtract is None else subtract
            c = c if c.numel() == 1 else (c.view(1, 1, -1) if c.numel() == v_pre.shape[2] else c.view(batch, 1, -1))
            if reset_mode == _lib.RESET_SUBTRACT:
                v_rec = v_pre - c * spikes
            else:
                v_rec = torch.where(spikes > 0, c.expand_as(v_pre), v_pre)
        return spikes, v_rec, v_post_last, count

    # ------------------------------------------------------------------
    # compact spike output (inference)
    _spike_dtype = torch.float32
    _spike_saturate = False

    def set_spike_output(self, dtype: torch.dtype = torch.float32, saturate: bool = False) -> "LIF":
        """Choose the element type of the layer's output raster.

        ``torch.float32`` (default) is the reference's format.  ``torch.uint8`` makes the forward kernel write one
        byte per neuron and step (3 of the forward's 12 bytes per neuron-step less on the way to a consumer that can
        take bytes) and, unless ``record_states`` is set, skip the membrane-potential tensor altogether.  Integer
        tensors carry no gradient, so this is for forward passes that are not differentiated: calling the layer with
        autograd recording raises.  Counts above 255 are stored as 255; with a spike function that allows more
        (``MultiSpike``, ``MaxSpike(k > 255)``) that must be accepted explicitly with ``saturate=True``.  The layer's
        state and ``firing_rate`` always use the true counts.
        """
        if dtype not in (torch.float32, torch.uint8):
            raise ValueError("spike output must be torch.float32 or torch.uint8")
        if dtype == torch.uint8:
            if self.spike_fn is None:
                raise ValueError("a non-spiking layer has no spike raster")
            k = self.max_num_spikes_per_bin
            if (k is None or k > 255) and not saturate:
                raise ValueError("this spike function can emit more than 255 spikes per step; pass saturate=True to "
                                 "store min(count, 255)")
        self._spike_dtype = dtype
        self._spike_saturate = bool(saturate)
        return self

    def _forward_compact(self, x: torch.Tensor, original_shape, has_synapse: bool):
        """Forward with the byte raster: straight to the library, no autograd node."""
        if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters())):
            raise ValueError("the uint8 spike output carries no gradient: call the layer under torch.no_grad() "
                             "(or set_spike_output(torch.float32) for training)")
        batch, time_steps, *trailing_dim = original_shape
        trailing = tuple(trailing_dim)
        dev = x.device
        B, T, M = x.shape
        N = B * M
        flat = lambda v: _flat32(_flat_param(v, trailing, batch, dev, self._perm))
        raw_mem, dmem = self._decay_source("mem")
        a_mem = flat(raw_mem)
        smem_flags = _lib.SCALE_ONE_MINUS_ALPHA if self.norm_input else 0
        th, lo = flat(self.spike_threshold), flat(self.min_v_mem)
        if isinstance(self.reset_fn, MembraneReset):
            reset_mode, c = _lib.RESET_TO_VALUE, flat(self.reset_fn.reset_value)
        else:
            reset_mode, c = _lib.RESET_SUBTRACT, flat(self.reset_fn.subtract_value)
        self._validate_once(dev)
        spec = lambda t, name, flags=0: (t, _mode_of(t, M, N, name) | flags)
        spikes = torch.empty((B, T, M), dtype=torch.uint8, device=dev)
        keep = bool(self.record_states)
        v_mem = torch.empty_like(x) if keep else None
        v_post_last = torch.empty(N, dtype=torch.float32, device=dev)
        count = torch.zeros(1, dtype=torch.int64, device=dev)
        v0 = self._state_flat(self.v_mem).to(torch.float32).contiguous()
        i_syn = None
        if has_synapse:
            raw_syn, dsyn = self._decay_source("syn")
            a_syn = flat(raw_syn)
            i_syn = torch.empty_like(x) if keep else None
            i_last = torch.empty(N, dtype=torch.float32, device=dev)
            i0 = self._state_flat(self.i_syn).to(torch.float32).contiguous()
            done = _lib.lif_syn_forward_u8(
                spikes, v_mem, i_syn, x, v0, i0, spec(a_syn, "alpha_syn", dsyn),
                spec(None, "scale_syn", _lib.SCALE_TIMES_ALPHA if self.decay_early else 0),
                spec(None, "scale_mem", smem_flags), spec(a_mem, "alpha_mem", dmem),
                spec(c, "subtract"), spec(th, "threshold"), spec(lo, "min_v_mem"), self.max_num_spikes_per_bin,
                reset_mode, self._spike_saturate, v_post_last, i_last, count, B, T, M)
        else:
            done = _lib.lif_forward_u8(
                spikes, v_mem, x, v0, spec(None, "in_scale", smem_flags), spec(a_mem, "alpha", dmem), spec(c, "subtract"),
                spec(th, "threshold"), spec(lo, "min_v_mem"), self.max_num_spikes_per_bin, reset_mode,
                self._spike_saturate, v_post_last, count, B, T, M)
        if not done:
            return None        # shape the byte kernels do not take: the caller converts the float raster
        if has_synapse:
            self._set_state("i_syn", self._unflatten(i_last, (batch,), trailing))
        self._set_state("v_mem", self._unflatten(v_post_last, (batch,), trailing))
        if keep:
            if i_syn is not None:
                self.recordings["i_syn"] = self._unflatten(i_syn, tuple(original_shape[:2]), tuple(original_shape[2:]))
            bc = lambda t: t if t.numel() == 1 else (t.view(1, 1, -1) if t.numel() == M else t.view(B, 1, -1))
            thb, cb = bc(th), bc(th if c is None else c)
            if reset_mode == _lib.RESET_SUBTRACT:       # true counts for the recording: rebuilt from v_mem, not from the bytes
                k = torch.where(v_mem >= thb, torch.div(v_mem, thb).trunc(), torch.zeros_like(v_mem))
                if self.max_num_spikes_per_bin is not None:
                    k = k.clamp(max=float(self.max_num_spikes_per_bin))
                v_rec = v_mem - cb * k
            else:
                v_rec = torch.where(spikes > 0, cb.expand_as(v_mem), v_mem)
            self.recordings["v_mem"] = self._unflatten(v_rec, tuple(original_shape[:2]), tuple(original_shape[2:]))
        out = self._unflatten(spikes, tuple(original_shape[:2]), tuple(original_shape[2:]))
        self._set_rate_source(count, out.numel())
        return out

    def _validate_once(self, dev) -> None:
        """Value checks of the reference Function (``spike.py:183,190``): 0 <= alpha <= 1 and
        threshold > min_v_mem.  Each check reads a result back from the GPU, which stalls the
        launch queue, so the outcome is remembered until one of the inputs changes."""
        def stamp(t):
            return (id(t), t._version) if isinstance(t, torch.Tensor) else t
        sources = [getattr(self, n, None) for n in ("tau_mem", "alpha_mem")]
        key = (str(dev),) + tuple(stamp(t) for t in sources) + (stamp(self.spike_threshold), stamp(self.min_v_mem))
        if getattr(self, "_validated_key", None) == key:
            return
        with torch.no_grad():
            a = torch.as_tensor(self._membrane_decay()[0]).detach().to(dev)
            bad, near_one = (((a < 0) | (a > 1)).any(), (a > 0.99).any())
            bad, near_one = torch.stack((bad, near_one)).tolist()      # one read-back for both
            if bad:
                raise ValueError("'alpha' must be between 0 and 1.")
            # 1 - alpha is the input scale under norm_input.  While it is at least 0.01 the backward rebuilds
            # the scale gradient from v_mem and need not keep or re-read the input; closer to zero it reads
            # the input.  The rebuilt term scale*x_t = v_t - alpha*vpost_{t-1} carries the rounding of v_t, at
            # most ulp(v_t)/2: an error of R_t*ulp(v_t)/(2*scale) per step with random sign, against the
            # R_t*vpost_{t-1} of the alpha gradient that it is combined with into the tau gradient, i.e.
            # 6e-8/scale <= 6e-6 of that per step before averaging over steps and neurons.  The decision is
            # taken from the parameter values seen here and is part of what a CUDA-graph capture freezes.
            self._scale_nonzero = not near_one
            if self.min_v_mem is not None:
                th = torch.as_tensor(self.spike_threshold, dtype=torch.float32, device=dev)
                lo = torch.as_tensor(self.min_v_mem, dtype=torch.float32, device=dev)
                if bool((th <= lo).any()):
                    raise ValueError("`threshold` must be greater than `min_v_mem`.")
        self.__dict__["_validated_key"] = key

    def forward(self, input_data: torch.Tensor):
        """``input_data``: (batch, time, ...) on a CUDA device.  Returns a tensor of the same shape."""
        x, original_shape = self._prepare_input(input_data)
        batch_size, time_steps, *trailing_dim = original_shape
        trailing = tuple(trailing_dim)
        self.__dict__["recordings"] = dict()

        has_synapse = getattr(self, "alpha_syn" if self.train_alphas else "tau_syn", None) is not None
        if self._spike_dtype == torch.uint8 and self.spike_fn is not None:
            out = self._forward_compact(x, original_shape, has_synapse) if time_steps > 0 and x.numel() > 0 else None
            if out is not None:
                return out
            # shapes the byte kernels do not take (neurons % 4 != 0, unaligned storage): float raster, converted
            with torch.no_grad():
                self._spike_dtype = torch.float32
                try:
                    out = self.forward(input_data)
                finally:
                    self._spike_dtype = torch.uint8
            return out.clamp(max=255.0).to(torch.uint8)
        if has_synapse and self.spike_fn is not None and fused_synaptic_eligible(x):
            return self._forward_fused_synaptic(x, original_shape)

        if not has_synapse:
            i_syn = x
        else:
            i_syn, i_last = self._forward_synaptic(x, batch_size, trailing)
            self._set_state("i_syn", self._unflatten(i_last, (batch_size,), trailing))
            if self.record_states:
                self.recordings["i_syn"] = self._unflatten(i_syn, tuple(original_shape[:2]), tuple(original_shape[2:]))

        output, v_rec, v_last, count = self._forward_membrane(i_syn, batch_size, trailing)
        if self.record_states:
            self.recordings["v_mem"] = self._unflatten(v_rec, tuple(original_shape[:2]), tuple(original_shape[2:]))
        self._set_state("v_mem", self._unflatten(v_last, (batch_size,), trailing))
        output_full = self._unflatten(output, tuple(original_shape[:2]), tuple(original_shape[2:]))
        # spike count (int64) or, for the non-spiking layer, the sum of the outputs (float64): both come
        # out of the forward kernel, so the reference's `output.sum() / numel` pass is not needed
        self._set_rate_source(count, output_full.numel(), output_full)
        return output_full

    def _forward_fused_synaptic(self, x: torch.Tensor, original_shape):
        """Synaptic and membrane stage in one kernel (same results as the two-stage route)."""
        batch_size, time_steps, *trailing_dim = original_shape
        trailing = tuple(trailing_dim)
        dev = x.device
        raw_syn, dsyn = self._decay_source("syn")
        raw_mem, dmem = self._decay_source("mem")
        raw_syn = _flat_param(raw_syn, trailing, batch_size, dev, self._perm)
        raw_mem = _flat_param(raw_mem, trailing, batch_size, dev, self._perm)
        flags = (dsyn, _lib.SCALE_TIMES_ALPHA if self.decay_early else 0,
                 dmem, _lib.SCALE_ONE_MINUS_ALPHA if self.norm_input else 0)
        use_acc = (raw_syn.requires_grad or raw_mem.requires_grad) and torch.is_grad_enabled()
        aux = self._aux(raw_mem.numel() + raw_syn.numel() if use_acc else 0, dev)
        acc = (aux[1:1 + raw_mem.numel()], aux[1 + raw_mem.numel():]) if use_acc else None
        threshold = _flat_param(self.spike_threshold, trailing, batch_size, dev, self._perm)
        min_v_mem = _flat_param(self.min_v_mem, trailing, batch_size, dev, self._perm)
        if isinstance(self.reset_fn, MembraneReset):
            reset_mode = _lib.RESET_TO_VALUE
            subtract = _flat_param(self.reset_fn.reset_value, trailing, batch_size, dev, self._perm)
        else:
            reset_mode = _lib.RESET_SUBTRACT
            subtract = _flat_param(self.reset_fn.subtract_value, trailing, batch_size, dev, self._perm)
        self._validate_once(dev)
        count = aux[:1].view(torch.int64)
        spikes, v_pre, v_post_last, i_syn, i_last = LIFSynapticTM.apply(
            x, raw_syn, None, self._state_flat(self.i_syn), raw_mem, None,
            self._state_flat(self.v_mem), threshold, subtract, min_v_mem, self.surrogate_grad_fn,
            self.max_num_spikes_per_bin, reset_mode, count, flags, acc,
            torch.is_grad_enabled() or self.record_states)      # inference without recording: spikes only
        self._set_state("i_syn", self._unflatten(i_last, (batch_size,), trailing))
        self._set_state("v_mem", self._unflatten(v_post_last, (batch_size,), trailing))
        if self.record_states:
            self.recordings["i_syn"] = self._unflatten(i_syn, tuple(original_shape[:2]), tuple(original_shape[2:]))
            c = threshold if subtract is None else subtract
            c = c if c.numel() == 1 else (c.view(1, 1, -1) if c.numel() == v_pre.shape[2] else c.view(batch_size, 1, -1))
            if reset_mode == _lib.RESET_SUBTRACT:
                v_rec = v_pre - c * spikes
            else:
                v_rec = torch.where(spikes > 0, c.expand_as(v_pre), v_pre)
            self.recordings["v_mem"] = self._unflatten(v_rec, tuple(original_shape[:2]), tuple(original_shape[2:]))
        output_full = self._unflatten(spikes, tuple(original_shape[:2]), tuple(original_shape[2:]))
        self._set_rate_source(count, output_full.numel(), output_full)
        return output_full

    # ``firing_rate`` (reference ``layers/lif.py:305``: mean of the output) is formed when it is read.  While the
    # caller still holds the output of a forward pass made with autograd on, it is the reference's differentiable
    # expression ``output.sum() / numel`` (a loss term on the rate gets its gradient); otherwise -- inference, or
    # the output already dropped -- it comes from the total that the forward kernel left on the device, which
    # costs no pass over the output and carries no graph.
    _rate_source = None
    _rate_value = None
    _rate_output = None

    def _set_rate_source(self, total: torch.Tensor, numel: int, output: Optional[torch.Tensor] = None) -> None:
        d = self.__dict__          # plain attributes: no need for nn.Module.__setattr__
        d["_rate_source"] = (total, max(int(numel), 1))
        d["_rate_value"] = None
        d["_rate_output"] = weakref.ref(output) if (output is not None and output.requires_grad) else None

    @property
    def firing_rate(self):
        if self._rate_value is None and self._rate_source is not None:
            total, numel = self._rate_source
            out = self._rate_output() if self._rate_output is not None else None
            if out is not None and torch.is_grad_enabled():
                self._rate_value = out.sum() / numel
            else:
                self._rate_value = total[0].to(torch.float32) / numel
        return self._rate_value

    @firing_rate.setter
    def firing_rate(self, value) -> None:
        self._rate_source = None
        self._rate_output = None
        self._rate_value = value

    def __repr__(self):
        return "EXODUS " + super().__repr__()
