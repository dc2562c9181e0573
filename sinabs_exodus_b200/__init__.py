"""B200-native implementation of the sinabs-exodus neuron path.

Public surface (same names as the reference's ``sinabs.exodus`` package):

* ``layers``      -- ``LIF``, ``IAF``, ``ExpLeak`` and their ``Squeeze`` variants
* ``spike``       -- ``IntegrateAndFire`` autograd Function
* ``leaky``       -- ``LeakyIntegrator`` autograd Function
* ``conversion``  -- ``sinabs_to_exodus``, ``exodus_to_sinabs``, ``module_map``

Beyond the reference: ``GraphedStep`` (``graphs``) captures a whole forward(+backward) step of a
network of these layers in a CUDA graph.

All computation runs in ``libexodus_b200.so`` (hand-written CUDA for sm_100a,
C ABI in ``include/exodus_b200.h``).  There is no PyTorch or CPU fallback: a
missing library or a CPU tensor raises.
"""
from __future__ import annotations

import sys as _sys

__version__ = "0.1.0"

from . import _lib  # noqa: E402
from . import leaky, spike  # noqa: E402
from . import layers  # noqa: E402
from . import conversion  # noqa: E402
from . import graphs  # noqa: E402
from .graphs import GraphedStep  # noqa: E402
from ._lib import device_status, set_nvtx_ranges, set_status_checks  # noqa: E402
from .leaky import LeakyIntegrator, LeakyIntegratorTM  # noqa: E402
from .spike import IntegrateAndFire, IntegrateAndFireTM, LIFSynapticTM  # noqa: E402


def install_as_sinabs_exodus() -> None:
    """Register this package under the module names of the reference plugin.

    After the call ``import sinabs.exodus.layers as el``, ``from sinabs.exodus.spike
    import IntegrateAndFire`` etc. resolve to this implementation, so code written
    against the reference runs unchanged.  Needs ``sinabs`` to be importable (the
    reference is a plugin inside the ``sinabs`` namespace).
    """
    import importlib

    importlib.import_module("sinabs")
    this = _sys.modules[__name__]
    _sys.modules["sinabs.exodus"] = this
    for name in ("layers", "spike", "leaky", "conversion"):
        _sys.modules[f"sinabs.exodus.{name}"] = getattr(this, name)
    _sys.modules["sinabs"].exodus = this
