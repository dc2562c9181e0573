"""Swap sinabs layers for EXODUS layers and back (reference ``sinabs/exodus/conversion.py:6-62``).

``module_map`` pairs each PyTorch-side layer class with its EXODUS counterpart.  The PyTorch-side
classes are ``sinabs.layers.*`` when sinabs is installed, else the parameter-and-state holders of
``sinabs_exodus_b200.compat.layers``.  A layer is rebuilt from its ``arg_dict`` (constructor
arguments including the current time constants and state shape), as the reference does.
"""
from __future__ import annotations

from typing import Iterable, Tuple

import torch

from . import layers as _exodus
from .compat import layers as _sinabs
from .compat.layers import replace_module

_LAYER_NAMES = ("IAF", "IAFSqueeze", "LIF", "LIFSqueeze", "ExpLeak", "ExpLeakSqueeze")

module_map = {getattr(_sinabs, name): getattr(_exodus, name) for name in _LAYER_NAMES}


def _swap(model: torch.nn.Module, pairs: Iterable[Tuple[type, type]]) -> torch.nn.Module:
    for source, target in pairs:
        def rebuild(layer, target=target):
            return target(**layer.arg_dict)
        model = replace_module(model, source, mapper_fn=rebuild)
    return model


def sinabs_to_exodus(model: torch.nn.Module) -> torch.nn.Module:
    """Every sinabs layer in ``model`` that has an EXODUS counterpart is replaced by it."""
    return _swap(model, module_map.items())


def exodus_to_sinabs(model: torch.nn.Module) -> torch.nn.Module:
    """Every EXODUS layer in ``model`` is replaced by the sinabs layer it stands in for."""
    return _swap(model, [(exodus_cls, sinabs_cls) for sinabs_cls, exodus_cls in module_map.items()])
