"""Fully asynchronous policy training: a rollouter thread keeps the servers saturated, a bounded message queue hands
finished prompt groups to the trainer, parameters are pushed every ``trigger_parameter_sync_step`` trainer steps, and
requests interrupted by a push resume with their partial output (partial rollout). Staleness is bounded: groups
older than ``staleness_threshold`` parameter versions are dropped.

Reference: ``verl/experimental/fully_async_policy/{fully_async_main,fully_async_rollouter,fully_async_trainer,
message_queue}.py``. Built here on the v1 pieces: the TransferQueue is the message queue, ``ReplayBufferAsync`` enforces
staleness, ``FullyAsyncLLMServerClient`` implements partial rollout.
"""

from __future__ import annotations

import threading
import time

from verl_b200.trainer.ppo.v1.replay_buffer import ReplayBufferAsync
from verl_b200.trainer.ppo.v1.trainer_base import PPOTrainer, _g, register_trainer

__all__ = ["FullyAsyncTrainer", "Rollouter"]


class Rollouter(threading.Thread):
    """Feeds prompts so that ready + in-flight prompt groups stay at ``max_queue_groups``; pauses while paused."""

    def __init__(self, trainer: "FullyAsyncTrainer", max_queue_groups: int, chunk: int):
        super().__init__(name="rollouter", daemon=True)
        self.trainer, self.max_queue_groups, self.chunk = trainer, max_queue_groups, chunk
        self._stop_evt, self._pause = threading.Event(), threading.Event()
        self.submitted_groups = 0

    def run(self):
        t = self.trainer
        while not self._stop_evt.is_set():
            if self._pause.is_set():
                time.sleep(0.002)
                continue
            groups = len({tags.get("uid") for tags in t.tq.kv_tags(t.partition_id).values()})
            if groups + self.chunk <= self.max_queue_groups:
                self.submitted_groups += t._submit_prompts(self.chunk * t.world)
            else:
                time.sleep(0.002)

    def pause(self):
        self._pause.set()

    def resume(self):
        self._pause.clear()

    def stop(self):
        self._stop_evt.set()


@register_trainer("fully_async")
class FullyAsyncTrainer(PPOTrainer):
    resumable_generation = True

    def _build_replay_buffer(self):
        a = _g(self.config, "async_training", None) or _g(self.config, "trainer.v1", {}) or {}
        self.staleness_threshold = int(a.get("staleness_threshold", 2))
        self.trigger_parameter_sync_step = int(a.get("trigger_parameter_sync_step", 1))
        self.partial_rollout = bool(a.get("partial_rollout", True))
        self.queue_batches = float(a.get("queue_batches", 2))
        return ReplayBufferAsync(self.tq, rollout_n=self.rollout_n, max_off_policy_threshold=self.staleness_threshold)

    def on_train_begin(self):
        per_rank = max(1, self.train_batch_size // self.world)
        self.rollouter = Rollouter(self, max_queue_groups=int(self.queue_batches * per_rank), chunk=max(1, per_rank // 4))
        self.rollouter.start()

    def on_step_begin(self):
        pass                                              # the rollouter feeds continuously

    def on_sample_end(self):
        # training is about to use the GPUs and then change the weights: stop feeding; with partial rollout also
        # interrupt what is running (it resumes under the new weights), otherwise let it drain
        self.rollouter.pause()
        if self.partial_rollout:
            self.agent_loop.abort()

    def on_step_end(self):
        self.agent_loop.server_manager.wake_up()
        self.rollouter.resume()

    def on_train_end(self):
        self.rollouter.stop()
        self.rollouter.join(timeout=10)
        super().on_train_end()
