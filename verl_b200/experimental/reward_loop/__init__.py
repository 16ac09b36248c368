from .reward_loop import RewardLoopManager, RewardLoopWorker, get_reward_loop_manager_cls, register_reward_loop
from .reward_model import RewardModelManager

__all__ = ["RewardLoopManager", "RewardLoopWorker", "RewardModelManager", "get_reward_loop_manager_cls", "register_reward_loop"]
