"""Decides whether a surrogate-gradient callable can be evaluated inside the backward kernel.

The reference evaluates ``surrogate_grad_fn(v_mem, threshold)`` with PyTorch and
hands the resulting tensor to its kernel (``spike.py:251``).  The fused backward
here computes three closed forms in registers (``EXB_SURR_*`` in
``include/exodus_b200.h``).  A callable is mapped to one of them only if it
*proves* to be that function: its class name and attributes propose a
candidate, and the candidate's formula is compared with the callable on a probe
grid of membrane potentials and thresholds.  Anything else -- an unknown
callable or a mismatch -- takes the generic route: the callable is evaluated
with PyTorch on the GPU and the kernel reads the tensor.  Both routes run the
same CUDA kernel family; neither is a CPU path.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

import torch

from . import _lib

_CACHE: Dict[Tuple, Tuple[int, float, float]] = {}


def _formula(kind: int, p0: float, p1: float, v: torch.Tensor, th: torch.Tensor) -> torch.Tensor:
    if kind == _lib.SURR_SINGLE_EXPONENTIAL:
        w = th * p0
        return p1 / w * torch.exp(-torch.abs(v - th) / w)
    if kind == _lib.SURR_HEAVISIDE:
        return (v >= (th - p0)).to(v.dtype) / th
    if kind == _lib.SURR_PERIODIC_EXPONENTIAL:
        half = th / 2
        u = v - half
        w = torch.where(v >= th, u - torch.floor(u / th), u)
        return p1 * torch.exp(-torch.abs(w - half) / p0) / th
    raise ValueError(kind)


def _candidate(fn: Callable):
    name = type(fn).__name__
    if name == "SingleExponential" and hasattr(fn, "grad_width"):
        return _lib.SURR_SINGLE_EXPONENTIAL, float(fn.grad_width), float(getattr(fn, "grad_scale", 1.0))
    if name == "Heaviside" and hasattr(fn, "window"):
        return _lib.SURR_HEAVISIDE, float(fn.window), 0.0
    if name == "PeriodicExponential" and hasattr(fn, "grad_width"):
        return _lib.SURR_PERIODIC_EXPONENTIAL, float(fn.grad_width), float(getattr(fn, "grad_scale", 1.0))
    return None


def _probe_matches(fn: Callable, kind: int, p0: float, p1: float) -> bool:
    # Thresholds and potentials that exercise both sides of the threshold, several
    # periods above it, and the edge of the Heaviside window.  Points that sit on
    # a discontinuity of the candidate are avoided by the irrational offsets.
    th = torch.tensor([0.3, 0.9, 1.0, 1.7], dtype=torch.float64).reshape(-1, 1)
    v = (torch.linspace(-3.0, 6.0, 181, dtype=torch.float64) + 0.00314159).reshape(1, -1)
    v = v.expand(th.shape[0], -1).contiguous()
    try:
        got = fn(v, th)
    except Exception:
        return False
    if not isinstance(got, torch.Tensor) or got.shape != v.shape:
        return False
    want = _formula(kind, p0, p1, v, th)
    return bool(torch.allclose(got.to(torch.float64), want, rtol=1e-6, atol=1e-9))


def classify(fn: Callable) -> Tuple[int, float, float]:
    """Return ``(kind, p0, p1)``; ``kind`` is ``SURR_GENERIC`` when the callable must be evaluated by PyTorch."""
    cand = _candidate(fn)
    if cand is None:
        return _lib.SURR_GENERIC, 0.0, 0.0
    key = (type(fn),) + cand
    if key not in _CACHE:
        _CACHE[key] = cand if _probe_matches(fn, *cand) else (_lib.SURR_GENERIC, 0.0, 0.0)
    return _CACHE[key]
