"""Swap sinabs layers for EXODUS layers and back (reference ``sinabs/exodus/conversion.py:6-62``).

``module_map`` pairs each PyTorch-side layer class with its EXODUS counterpart.
The PyTorch-side classes are ``sinabs.layers.*`` when sinabs is installed, else
the parameter-and-state holders of ``sinabs_exodus_b200.compat.layers``.
"""
from __future__ import annotations

import torch

from . import layers as el
from .compat import layers as sl
from .compat.layers import replace_module

module_map = {
    sl.IAF: el.IAF,
    sl.IAFSqueeze: el.IAFSqueeze,
    sl.LIF: el.LIF,
    sl.LIFSqueeze: el.LIFSqueeze,
    sl.ExpLeak: el.ExpLeak,
    sl.ExpLeakSqueeze: el.ExpLeakSqueeze,
}


def exodus_to_sinabs(model: torch.nn.Module):
    """Replace all EXODUS layers with their sinabs equivalents; layer attributes are copied over."""
    mapping_list = [
        (exodus_class, lambda module, replacement=sinabs_class: replacement(**module.arg_dict))
        for sinabs_class, exodus_class in module_map.items()
    ]
    for class_to_replace, mapper_fn in mapping_list:
        model = replace_module(model, class_to_replace, mapper_fn=mapper_fn)
    return model


def sinabs_to_exodus(model: torch.nn.Module):
    """Replace all sinabs layers with their EXODUS equivalents; layer attributes are copied over."""
    mapping_list = [
        (sinabs_class, lambda module, replacement=exodus_class: replacement(**module.arg_dict))
        for sinabs_class, exodus_class in module_map.items()
    ]
    for class_to_replace, mapper_fn in mapping_list:
        model = replace_module(model, class_to_replace, mapper_fn=mapper_fn)
    return model
