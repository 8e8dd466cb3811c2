from .communicator import CollectiveError, CollInfo, Communicator, FLAG_MUTE_SENDS, FLAG_ROUND_EACH_ADD

__all__ = ["Communicator", "CollInfo", "CollectiveError", "FLAG_MUTE_SENDS", "FLAG_ROUND_EACH_ADD"]
