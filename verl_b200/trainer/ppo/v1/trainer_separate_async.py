"""Separate asynchronous v1 trainer: rollout replicas live on their OWN GPUs (standalone server processes), training on the
rest; generation never stops for training.

* The rollout pool is a set of ``RolloutReplica`` server processes — started here on ``trainer.v1.rollout_devices`` (CUDA
  device ids; one process each) or attached to through ``trainer.v1.rollout_addresses`` (``host:port`` of servers started by
  ``python -m verl_b200.workers.rollout.replica``).
* Prompts are streamed to the pool (``async_warmup_batches`` ahead, one more batch per step); finished trajectories land in
  the TransferQueue; the replay buffer hands whole prompt groups to the trainer and evicts groups older than
  ``max_off_policy_threshold`` steps.
* After every update the trainer ranks push the new weights to the replicas (rank r serves replicas r, r + world, …): the
  engine exposes its bf16 parameter buffer through a CUDA IPC handle and the replica copies it device-to-device over NVLink
  (a file on CPU). Requests interrupted by the hand-off are resumed by the clients with the tokens they already have
  (partial rollout), so a trajectory may span weight versions.

Reference: ``verl/trainer/ppo/v1/trainer_separate_async.py:46`` (disjoint trainer / rollouter GPU pools, parameter
synchronisation through the checkpoint engine, staleness control).
"""

from __future__ import annotations

import os
import tempfile

from verl_b200.workers.rollout.llm_server import LLMServerManager
from verl_b200.workers.rollout.replica import RolloutMode, RolloutReplica

from .agent_loop_tq import AgentLoopManagerTQ
from .checkpoint_callback import CheckpointCallback
from .replay_buffer import ReplayBufferAsync
from .trainer_base import PPOTrainer, _g, register_trainer

__all__ = ["PPOTrainerSeparateAsync"]


@register_trainer("separate_async")
class PPOTrainerSeparateAsync(PPOTrainer):
    resumable_generation = True

    def _build_replay_buffer(self):
        a = _g(self.config, "trainer.v1", {}) or {}
        self.async_warmup_batches = float(a.get("async_warmup_batches", 1))
        fg = _g(self.config, "algorithm.filter_groups", {}) or {}
        return ReplayBufferAsync(self.tq, rollout_n=self.rollout_n, filter_groups=bool(fg.get("enable", False)),
                                 filter_metric=fg.get("metric", "score") or "score",
                                 max_off_policy_threshold=int(a.get("max_off_policy_threshold", 2)))

    # ------------------------------------------------------------------ rollout pool
    def _start_pool(self) -> list[RolloutReplica]:
        a = _g(self.config, "trainer.v1", {}) or {}
        ro = self.config.actor_rollout_ref.rollout
        addresses = list(a.get("rollout_addresses", None) or [])
        self._owned: list[RolloutReplica] = []
        if not addresses and self.rank == 0:
            devices = a.get("rollout_devices", None)
            devices = [None] if devices in (None, "", []) else [str(d) for d in (devices if isinstance(devices, (list, tuple)) else str(devices).split(","))]
            model = _g(self.config, "actor_rollout_ref.model.path", None) or _g(self.config, "actor_rollout_ref.model.preset", None)
            max_len = int(self.config.data.max_prompt_length) + int(self.config.data.max_response_length) + 8
            extra = ["--max-num-seqs", str(int(_g(ro, "max_num_seqs", 256))), "--max-model-len", str(int(_g(ro, "max_model_len", None) or max_len)),
                     "--gpu-memory-utilization", str(float(a.get("rollout_gpu_memory_utilization", 0.85)))]
            if a.get("rollout_num_blocks", None):
                extra += ["--num-blocks", str(int(a["rollout_num_blocks"]))]
            for i, dev in enumerate(devices):
                r = RolloutReplica(i, ro, mode=RolloutMode.STANDALONE).init_standalone(str(model), device=dev, extra_args=extra)
                self._owned.append(r)
                addresses.append(r.address)
        if self.world > 1:
            import torch.distributed as dist

            from verl_b200.single_controller.spmd import init_spmd_process_group

            box = [addresses]
            dist.broadcast_object_list(box, src=0, group=init_spmd_process_group())
            addresses = box[0]
        owned = {r.address: r for r in self._owned}
        return [owned.get(ad) or RolloutReplica(i, ro, mode=RolloutMode.STANDALONE).init_remote(ad) for i, ad in enumerate(addresses)]

    def _setup(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = self.stages.actor_rollout_wg.world_size
        worker = self.stages.actor_rollout_wg.worker
        local = worker._agent_loop_manager()                   # tokenizer and tools of the colocated stack; its engine stays asleep
        self.replicas = self._start_pool()
        servers = LLMServerManager(self.replicas, fully_async=True)
        self.agent_loop = AgentLoopManagerTQ(self.config.actor_rollout_ref, servers, local.tokenizer, tools=local.workers[0].tools,
                                             reward_fn=None, tq=self.tq, partition_id=self.partition_id)
        self.replay_buffer = self._build_replay_buffer()
        self.checkpoint_callback = CheckpointCallback(self.config.trainer)
        self.param_version = 0
        self._export_file = None

    # ------------------------------------------------------------------ weight hand-off
    def sync_weights(self) -> dict:
        """Push the trainer's current weights to the replicas this rank serves."""
        import time

        t0 = time.perf_counter()
        engine = self.stages.actor_rollout_wg.worker.actor.engine
        mine = [r for i, r in enumerate(self.replicas) if i % self.world == self.rank]
        versions = []
        if mine:
            if engine.store.flat.is_cuda:
                src = engine.export_weights_source()
            else:
                if self._export_file is None:
                    self._export_file = os.path.join(tempfile.mkdtemp(prefix="verl_b200_weights_"), f"rank{self.rank}.pt")
                src = engine.export_weights_source(self._export_file)
            versions = [r.update_weights(src) for r in mine]
        self.param_version += 1
        return {"sync/weights_s": time.perf_counter() - t0, "sync/param_version": self.param_version,
                "sync/replica_version_min": min(versions) if versions else self.param_version}

    # ------------------------------------------------------------------ hooks
    def on_train_begin(self):
        self.sync_weights()                   # the pool starts from the trainer's weights, whatever the servers loaded
        n = int(round(self.async_warmup_batches * self.train_batch_size))
        if n > 0:
            self._submit_prompts(n)

    def on_step_begin(self):
        self._submit_prompts(self.train_batch_size)

    def on_sample_begin(self):
        need = max(1, self.train_batch_size // self.world)
        self.replay_buffer.wait_for_sampleable(self.global_steps, self.partition_id, need)

    def step(self, metrics: dict, timing_raw: dict):
        out = super().step(metrics, timing_raw)
        metrics.update(self.sync_weights())
        return out

    def on_train_end(self):
        self.agent_loop.shutdown()
        for r in getattr(self, "_owned", []):
            r.shutdown()
        if self._export_file and os.path.exists(self._export_file):
            os.unlink(self._export_file)
