"""The EXODUS layers: ``LIF`` and the variants derived from it."""
from .lif import LIF
from .variants import IAF, ExpLeak, ExpLeakSqueeze, IAFSqueeze, LIFSqueeze

__all__ = ["LIF", "LIFSqueeze", "IAF", "IAFSqueeze", "ExpLeak", "ExpLeakSqueeze"]
