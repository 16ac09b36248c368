from .managers import DAPORewardLoopManager, GDPORewardLoopManager, NaiveRewardLoopManager, RateLimitedRewardLoopManager, RemoteRewardLoopManager

__all__ = ["NaiveRewardLoopManager", "DAPORewardLoopManager", "GDPORewardLoopManager", "RateLimitedRewardLoopManager", "RemoteRewardLoopManager"]
