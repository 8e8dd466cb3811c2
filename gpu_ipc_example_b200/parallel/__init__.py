from .communicator import CollectiveError, CollInfo, Communicator, FLAG_MUTE_SENDS, FLAG_ROUND_EACH_ADD

from .layers import ColumnParallelLinear, RowParallelLinear

__all__ = ["ColumnParallelLinear", "RowParallelLinear", "Communicator", "CollInfo", "CollectiveError", "FLAG_MUTE_SENDS", "FLAG_ROUND_EACH_ADD"]
