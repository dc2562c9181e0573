from .lif import LIF, LIFSqueeze
from .iaf import IAF, IAFSqueeze
from .exp_leak import ExpLeak, ExpLeakSqueeze

__all__ = ["LIF", "LIFSqueeze", "IAF", "IAFSqueeze", "ExpLeak", "ExpLeakSqueeze"]
