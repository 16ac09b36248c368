"""On-policy v1 trainer: one batch is generated, awaited and trained on per step
(reference: ``verl/trainer/ppo/v1/trainer_sync.py:24``)."""

from __future__ import annotations

from .trainer_base import PPOTrainer, register_trainer

__all__ = ["PPOTrainerSync"]


@register_trainer("sync")
class PPOTrainerSync(PPOTrainer):
    def on_step_begin(self):
        self._submit_prompts(self.train_batch_size)
