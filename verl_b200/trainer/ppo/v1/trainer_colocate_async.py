"""Colocated asynchronous v1 trainer: rollout and training share the GPUs in time slices, generation runs ahead.

``async_warmup_batches`` extra batches are submitted before the first step so the servers always have work; each step
submits one more. Sampling starts as soon as ``switch_threshold`` × the needed prompt groups are ready: whatever is still
generating is interrupted (clients resume those requests after the weight update with the tokens they already have), so
the long tail of a batch no longer idles the GPUs. Groups that fall more than ``max_off_policy_threshold`` steps behind
are evicted by the replay buffer. Reference: ``verl/trainer/ppo/v1/trainer_colocate_async.py`` (hybrid GPU lending with
an adaptive switch threshold).
"""

from __future__ import annotations

import time

from .replay_buffer import ReplayBufferAsync
from .trainer_base import PPOTrainer, _g, register_trainer

__all__ = ["PPOTrainerColocateAsync"]


@register_trainer("colocate_async")
class PPOTrainerColocateAsync(PPOTrainer):
    resumable_generation = True

    def _build_replay_buffer(self):
        a = _g(self.config, "trainer.v1", {}) or {}
        self.async_warmup_batches = float(a.get("async_warmup_batches", 1))
        self.switch_threshold = float(a.get("switch_threshold", 1.0))
        fg = _g(self.config, "algorithm.filter_groups", {}) or {}
        return ReplayBufferAsync(self.tq, rollout_n=self.rollout_n, filter_groups=bool(fg.get("enable", False)),
                                 filter_metric=fg.get("metric", "score") or "score",
                                 max_off_policy_threshold=int(a.get("max_off_policy_threshold", 1)))

    def on_train_begin(self):
        n = int(round(self.async_warmup_batches * self.train_batch_size))
        if n > 0:
            self._submit_prompts(n)

    def on_step_begin(self):
        self._submit_prompts(self.train_batch_size)

    def on_sample_begin(self):
        need = max(1, self.train_batch_size // self.world)
        self.replay_buffer.wait_for_sampleable(self.global_steps, self.partition_id, need)
        if self.switch_threshold < 1.0 or self.agent_loop.inflight > 0:
            # hand the GPUs to training: stop generation now, unfinished requests continue after the update
            self.agent_loop.abort()

    def on_step_end(self):
        self.agent_loop.server_manager.wake_up()
