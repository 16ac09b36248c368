"""v1 trainers: generation is decoupled from training through the TransferQueue and a replay buffer.

Data flow: prompts → ``AgentLoopManagerTQ.submit`` (server-mode rollout, returns immediately) → finished trajectories
land in the queue → ``ReplayBuffer.sample`` picks whole prompt groups → the usual PPO stages (reward, old/ref log-prob,
values, advantages, updates) → weight hand-off. Subclasses decide how far generation may run ahead of training:

* ``PPOTrainerSync``            on-policy: submit one batch, wait for it, train;
* ``PPOTrainerSeparateAsync``   rollout replicas on their own GPUs (server processes); weights are pushed after every update;
* ``PPOTrainerColocateAsync``   keeps ``async_warmup_batches`` batches in flight on the shared GPUs; when
                                ``switch_threshold`` of the needed groups are ready the rest is interrupted and resumed
                                after the update (partial rollout), stale groups are evicted.

Reference: ``verl/trainer/ppo/v1/trainer_base.py:113-2021`` (``PPOTrainer`` with ``_setup / fit / step / _step_once`` and
``on_*`` hooks, trainer registry), ``trainer_sync.py:24``, ``trainer_colocate_async.py``.
"""

from __future__ import annotations

import os
import time
import uuid
from abc import ABC, abstractmethod
from typing import Optional

import numpy as np

from verl_b200.protocol import DataProto
from verl_b200.trainer.ppo.metric_utils import compute_throughout_metrics, compute_timing_metrics
from verl_b200.trainer.ppo.ppo_trainer import PPOTrainer as _StageTrainer
from verl_b200.trainer.ppo.ppo_trainer import marked_timer
from verl_b200.trainer.ppo.v1.agent_loop_tq import AgentLoopManagerTQ
from verl_b200.trainer.ppo.v1.checkpoint_callback import CheckpointCallback
from verl_b200.trainer.ppo.v1.replay_buffer import ReplayBuffer, ReplayBufferAsync
from verl_b200.utils.tracking import Tracking
from verl_b200.utils.transfer_queue import TransferQueue

__all__ = ["PPOTrainer", "register_trainer", "get_trainer_cls"]

_TRAINERS: dict[str, type] = {}


def register_trainer(name: str):
    def deco(cls):
        _TRAINERS[name] = cls
        return cls

    return deco


def get_trainer_cls(name: str):
    if name not in _TRAINERS:
        from . import trainer_colocate_async, trainer_separate_async, trainer_sync  # noqa: F401

    if name not in _TRAINERS:
        raise ValueError(f"unknown v1 trainer {name!r}; known: {sorted(_TRAINERS)}")
    return _TRAINERS[name]


def _g(cfg, path, default=None):
    cur = cfg
    for p in path.split("."):
        if cur is None:
            return default
        cur = cur.get(p, None) if hasattr(cur, "get") else getattr(cur, p, None)
    return default if cur is None else cur


class PPOTrainer(ABC):
    partition_id = "train"
    resumable_generation = False     # async trainers interrupt generation and let the clients resume it

    def __init__(self, config, tokenizer=None, reward_fn=None, val_reward_fn=None, train_dataset=None, val_dataset=None):
        self.config = config
        self.stages = _StageTrainer(config, tokenizer=tokenizer, reward_fn=reward_fn, val_reward_fn=val_reward_fn,
                                    train_dataset=train_dataset, val_dataset=val_dataset)
        self.tokenizer = tokenizer
        self.global_steps = 0
        self.tq = TransferQueue()
        self.rollout_n = int(config.actor_rollout_ref.rollout.n)
        self.train_batch_size = int(config.data.train_batch_size)
        self._data_iter = None
        self._epoch = 0

    # ------------------------------------------------------------------ set-up
    def init(self):
        self.stages.init_workers()
        self._setup()
        self.on_init_end()

    def _build_replay_buffer(self) -> ReplayBuffer:
        fg = _g(self.config, "algorithm.filter_groups", {}) or {}
        return ReplayBuffer(self.tq, rollout_n=self.rollout_n, filter_groups=bool(fg.get("enable", False)),
                            filter_metric=fg.get("metric", "score") or "score")

    def _setup(self):
        worker = self.stages.actor_rollout_wg.worker      # in-process worker of the SPMD backend
        mgr = worker._agent_loop_manager()
        from verl_b200.workers.rollout.llm_server import LLMServerManager

        servers = LLMServerManager(mgr.server_manager.replicas, fully_async=self.resumable_generation)
        self.agent_loop = AgentLoopManagerTQ(self.config.actor_rollout_ref, servers, mgr.tokenizer, tools=mgr.workers[0].tools,
                                             reward_fn=None, tq=self.tq, partition_id=self.partition_id)
        self.replay_buffer = self._build_replay_buffer()
        self.checkpoint_callback = CheckpointCallback(self.config.trainer)
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = self.stages.actor_rollout_wg.world_size

    # ------------------------------------------------------------------ data
    def _next_prompts(self, num_prompts: int) -> DataProto:
        rows = []
        have = 0
        while have < num_prompts:
            if self._data_iter is None:
                self._data_iter = iter(self.stages.train_dataloader)
            try:
                b = DataProto.from_single_dict(next(self._data_iter))
            except StopIteration:
                self._data_iter, self._epoch = None, self._epoch + 1
                continue
            rows.append(b)
            have += len(b)
        batch = DataProto.concat(rows)[:num_prompts]
        batch.non_tensor_batch["uid"] = np.array([str(uuid.uuid4()) for _ in range(len(batch))], dtype=object)
        return batch

    def _submit_prompts(self, num_prompts: int) -> int:
        """Each controller rank rolls out its share of the prompts on its own replica."""
        batch = self._next_prompts(num_prompts)
        mine = batch[self.rank:: self.world] if self.world > 1 else batch
        mine.meta_info = self.stages._gen_meta()
        mine.meta_info["global_steps"] = self.global_steps
        self.agent_loop.submit(mine, gen_step=self.global_steps, n=self.rollout_n)
        return len(mine)

    def _materialize(self, meta) -> DataProto:
        batch = self.tq.kv_get(meta)
        if self.world > 1:
            import torch.distributed as dist

            from verl_b200.single_controller.spmd import init_spmd_process_group

            parts = [None] * self.world
            dist.all_gather_object(parts, batch, group=init_spmd_process_group())
            batch = DataProto.concat(parts)
        return batch

    # ------------------------------------------------------------------ loop
    def fit(self):
        cfg = self.config
        logger = Tracking(cfg.trainer.project_name, cfg.trainer.experiment_name, cfg.trainer.logger if self.rank == 0 else [], config=dict(cfg))
        self.global_steps = self.stages._load_checkpoint() or 0
        self.stages.global_steps = self.global_steps
        if self.global_steps:
            self.stages.actor_rollout_wg.update_weights()      # the colocated rollout must serve the restored weights
        total = int(self.stages.total_training_steps)
        self.on_train_begin()
        while self.global_steps < total:
            self.global_steps += 1
            self.stages.global_steps = self.global_steps
            metrics, timing_raw = {}, {}
            self.on_step_begin()
            t0 = time.perf_counter()
            with marked_timer("step", timing_raw):
                self.step(metrics, timing_raw)
            self.on_step_end()
            is_last = self.global_steps >= total
            if self.stages.val_reward_fn is not None and int(_g(cfg, "trainer.test_freq", -1)) > 0 and \
                    (is_last or self.global_steps % int(cfg.trainer.test_freq) == 0):
                self.on_validate_begin()
                metrics.update(self.stages._validate())
                self.on_validate_end()
            if self.checkpoint_callback.should_save(self.global_steps, is_last, time.perf_counter() - t0):
                self.stages._save_checkpoint()
            metrics.update({"training/global_step": self.global_steps, "training/epoch": self._epoch})
            logger.log(data=metrics, step=self.global_steps)
            self.stages._finish_pending_checkpoint(block=False)
        self.stages._finish_pending_checkpoint(block=True)
        self.on_train_end()

    def step(self, metrics: dict, timing_raw: dict):
        return self._step_once(metrics, timing_raw, self.train_batch_size)

    def _step_once(self, metrics: dict, timing_raw: dict, sample_batch_size: int):
        self.on_sample_begin()
        with marked_timer("gen", timing_raw):
            meta, rb_metrics = self.replay_buffer.sample(self.global_steps, self.partition_id, max(1, sample_batch_size // self.world))
        self.on_sample_end()
        metrics.update(rb_metrics)
        batch = self._materialize(meta)
        self.replay_buffer.release(meta)
        batch.meta_info = {}
        metrics.update(self.stages.train_on_rollouts(batch, timing_raw, self.rollout_n))
        last = self.stages._last_batch
        metrics.update(compute_timing_metrics(batch=last, timing_raw=timing_raw))
        metrics.update(compute_throughout_metrics(batch=last, timing_raw={**timing_raw, "step": sum(v for k, v in timing_raw.items() if k in ("gen", "train"))},
                                                  n_gpus=max(1, self.world)))
        return meta

    # ------------------------------------------------------------------ hooks
    def on_init_end(self):
        pass

    def on_train_begin(self):
        pass

    def on_train_end(self):
        self.agent_loop.shutdown()
        self.agent_loop.server_manager.shutdown()

    def on_validate_begin(self):
        pass

    def on_validate_end(self):
        pass

    @abstractmethod
    def on_step_begin(self):
        ...

    def on_step_end(self):
        pass

    def on_sample_begin(self):
        pass

    def on_sample_end(self):
        pass
