"""When to checkpoint (reference: ``verl/trainer/ppo/checkpoint_callback.py:33-82``): every ``save_freq`` steps, on the
last step, and when the announced end of the machine reservation is closer than one step plus a safety margin."""

from __future__ import annotations

from verl_b200.utils.checkpoint.checkpoint_manager import should_save_ckpt_esi

__all__ = ["CheckpointCallback"]


class CheckpointCallback:
    def __init__(self, trainer_config):
        get = trainer_config.get if hasattr(trainer_config, "get") else lambda k, d=None: getattr(trainer_config, k, d)
        self.save_freq = int(get("save_freq", -1) or -1)
        self.esi_redundant_time = float(get("esi_redundant_time", 0) or 0)
        self.max_step_time = 0.0

    def should_save(self, global_step: int, is_last_step: bool, step_time_s: float = 0.0) -> bool:
        self.max_step_time = max(self.max_step_time, step_time_s)
        if self.save_freq <= 0:
            return False
        if is_last_step or global_step % self.save_freq == 0:
            return True
        return should_save_ckpt_esi(self.max_step_time, redundant_time=self.esi_redundant_time)
