"""Stand-ins for the parts of the ``sinabs`` package that the exodus layers touch.

The reference layers subclass ``sinabs.layers.LIF`` and take their activation
tokens and surrogate-gradient callables from ``sinabs.activation``.  When
``sinabs`` can be imported, its objects are used and the layers here subclass
the real base class, so ``state_dict`` and ``conversion`` interoperate with it.
When it cannot, the small classes in this sub-package provide the same surface
(names, constructor arguments, attributes), written from the way the reference
layers and tests use them.
"""
from __future__ import annotations

try:  # pragma: no cover - depends on the environment
    import sinabs  # noqa: F401
    import sinabs.layers  # noqa: F401
    import sinabs.activation  # noqa: F401
    HAVE_SINABS = True
except Exception:  # ImportError or a broken install
    HAVE_SINABS = False
