"""One-step-off-policy training: the batch for step t+1 is generated with the weights of step t−1 while step t trains,
so rollout and training overlap at the price of one step of staleness and nothing is ever interrupted
(reference: ``verl/experimental/one_step_off_policy/ray_trainer.py:49``)."""

from verl_b200.trainer.ppo.v1.replay_buffer import ReplayBufferAsync
from verl_b200.trainer.ppo.v1.trainer_base import PPOTrainer, _g, register_trainer

__all__ = ["OneStepOffPolicyTrainer"]


@register_trainer("one_step_off_policy")
class OneStepOffPolicyTrainer(PPOTrainer):
    def _build_replay_buffer(self):
        fg = _g(self.config, "algorithm.filter_groups", {}) or {}
        return ReplayBufferAsync(self.tq, rollout_n=self.rollout_n, filter_groups=bool(fg.get("enable", False)),
                                 filter_metric=fg.get("metric", "score") or "score", max_off_policy_threshold=1)

    def on_train_begin(self):
        self._submit_prompts(self.train_batch_size)       # the batch step 1 will train on

    def on_step_begin(self):
        self._submit_prompts(self.train_batch_size)       # generated while this step trains; consumed by the next
