"""b200ipc: single-kernel intra-node collectives for B200 (sm_100a, NVLink 5 / NVSwitch),
fused with the compute that surrounds them in tensor-parallel inference."""
from .parallel import CollectiveError, CollInfo, Communicator

__all__ = ["Communicator", "CollInfo", "CollectiveError"]
__version__ = "0.1.0"
