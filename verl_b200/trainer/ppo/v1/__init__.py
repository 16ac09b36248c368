from .replay_buffer import ReplayBuffer, ReplayBufferAsync
from .trainer_base import PPOTrainer, get_trainer_cls, register_trainer
from .trainer_colocate_async import PPOTrainerColocateAsync
from .trainer_sync import PPOTrainerSync

__all__ = ["PPOTrainer", "PPOTrainerSync", "PPOTrainerColocateAsync", "ReplayBuffer", "ReplayBufferAsync", "get_trainer_cls", "register_trainer"]
