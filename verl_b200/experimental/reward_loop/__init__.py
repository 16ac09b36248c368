from .reward_loop import RewardLoopManager, RewardLoopWorker, get_reward_loop_manager_cls, register_reward_loop

__all__ = ["RewardLoopManager", "RewardLoopWorker", "get_reward_loop_manager_cls", "register_reward_loop"]
