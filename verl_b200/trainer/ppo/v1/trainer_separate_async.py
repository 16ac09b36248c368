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

* Lending (``trainer.v1.separate_async.hybrid_rollout.enable_switch``): while the trainer would only wait for trajectories its
  own GPUs serve generation too. The colocated engine of the training rank joins the balancer after a step ("rollout" mode) and
  is taken back, with its open requests handed to the pool as partial rollouts, once ``switch_threshold_ratio`` of the next
  batch is sampleable ("trainer" mode). The threshold adapts: it rises after steps that still idled, falls after calm ones; a
  switch is only made when the wait it is expected to save exceeds the measured cost of switching there and back.

Reference: ``verl/trainer/ppo/v1/trainer_separate_async.py:40-420`` (disjoint trainer / rollouter GPU pools, parameter
synchronisation through the checkpoint engine, staleness control, ``HybridEngineMode`` switching).
"""

from __future__ import annotations

import enum
import os
import tempfile
import time
from collections import deque

from verl_b200.workers.rollout.llm_server import LLMServerManager
from verl_b200.workers.rollout.replica import RolloutMode, RolloutReplica

from .agent_loop_tq import AgentLoopManagerTQ
from .checkpoint_callback import CheckpointCallback
from .replay_buffer import ReplayBufferAsync
from .trainer_base import PPOTrainer, _g, register_trainer

__all__ = ["PPOTrainerSeparateAsync", "HybridEngineMode"]


class HybridEngineMode(enum.Enum):
    TRAINER = "trainer"
    ROLLOUT = "rollout"


class _Lender:
    """What the dynamic-schedule controller drives: the trainer's two mode switches and the balancer's sticky-session table."""

    def __init__(self, trainer: "PPOTrainerSeparateAsync"):
        self.t = trainer

    def activate(self):
        self.t.switch_to_rollout()

    def deactivate(self):
        self.t.switch_to_trainer()

    def rebalance(self):
        """Forget which server each open conversation was pinned to, so that follow-up turns go to the least-loaded server —
        the engines that just joined start empty."""
        bal = getattr(self.t._servers, "balancer", None)
        n = len(bal.sticky) if bal is not None else 0
        if bal is not None:
            bal.sticky.clear()
        return {"cleared_entries": n}


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
        self._setup_hybrid(local, servers)

    # ------------------------------------------------------------------ lending the training GPUs to generation
    def _setup_hybrid(self, local, servers: LLMServerManager):
        from verl_b200.trainer.config import HybridRolloutSwitchConfig

        raw = dict(_g(self.config, "trainer.v1.separate_async.hybrid_rollout", {}) or {})
        known = {f for f in HybridRolloutSwitchConfig.__dataclass_fields__}
        self.hybrid_rollout_config = HybridRolloutSwitchConfig(**{k: v for k, v in raw.items() if k in known})
        self.current_mode = HybridEngineMode.TRAINER
        self._servers = servers
        self._hybrid_replica = None
        self.parameter_sync_step = int(_g(self.config, "trainer.v1.separate_async.parameter_sync_step", 1) or 1)
        enable = bool(_g(self.config, "actor_rollout_ref.hybrid_engine", True)) and self.hybrid_rollout_config.enable_switch
        if self.hybrid_rollout_config.enable_switch and not enable:
            print("[separate_async] hybrid_rollout.enable_switch is ignored because actor_rollout_ref.hybrid_engine=False", flush=True)
        self._switch_enabled = enable
        if not enable:
            return
        self._hybrid_replica = local.server_manager.replicas[0]            # the colocated engine of this training rank
        self._hybrid_name = f"hybrid-{self.rank}"
        c = self.hybrid_rollout_config
        self._switch_threshold_ratio = float(c.switch_threshold_ratio)
        self._idle_steps = self._calm_steps = 0
        self._step_sample_wait_seconds = 0.0
        self._step_wait_samples = 0
        self._wait_seconds = 0.0
        self._wait_samples = 0
        self._to_rollout_costs: deque = deque(maxlen=int(c.switch_cost_window_size))
        self._to_trainer_costs: deque = deque(maxlen=int(c.switch_cost_window_size))
        standalone = max(1, len(self.replicas))
        self._scaling_factor = (self.world + standalone) / standalone          # generation capacity with / without the lent GPUs
        self.switch_log: list = []
        self._consumed_groups = 0
        self._controller = None
        if c.policy:
            from verl_b200.experimental.fully_async_policy.dynamic_schedule import DynamicResourceController

            kw = dict(c.policy_kwargs or {})
            kw.setdefault("deactivate_ratio", float(c.switch_threshold_ratio))
            self._controller = DynamicResourceController(_Lender(self), num_standalone_replicas=len(self.replicas), num_hybrid_replicas=self.world,
                                                         policy=str(c.policy), policy_kwargs=kw)

    def _schedule_context(self, next_step: int):
        """What the lending policy sees, with every number agreed across the training ranks. Units are prompt groups: one
        collection is one mini-batch, one cycle (``parameter_sync_step`` collections) is one training batch."""
        from verl_b200.experimental.fully_async_policy.dynamic_schedule import DynamicScheduleContext

        mini = max(1, self.train_batch_size // self.parameter_sync_step)
        ready = self._sampleable(next_step)
        wait_s = self._agree(self._step_sample_wait_seconds, "max")
        wait_n = int(self._agree(float(self._step_wait_samples), "max")) * self.world
        poll = max(5.0 * float(getattr(self.replay_buffer, "poll_interval_s", 0.01)), 0.05)
        waited = wait_s > poll and wait_n > 0
        ctl = self._controller
        ctx = DynamicScheduleContext(required_samples=mini, trigger_parameter_sync_step=self.parameter_sync_step,
                                     total_generated_samples=self._consumed_groups + ready, expected_samples=self._consumed_groups,
                                     buffer_samples=int(getattr(self.replay_buffer, "max_off_policy_threshold", 1) or 1) * self.train_batch_size,
                                     step_wait_times=[wait_s] if waited else [], step_wait_samples=[wait_n] if waited else [])
        ctx.last_activate_duration_s = self._agree(ctl.last_activate_duration_s, "max")
        ctx.last_deactivate_duration_s = self._agree(ctl.last_deactivate_duration_s, "max")
        return ctx

    def _take_back(self):
        if self._controller is not None:
            self._controller.deactivate(self.global_steps)
        else:
            self.switch_to_trainer()

    def _agree(self, value: float, op: str) -> float:
        """The controller runs on every rank; decisions that change collective behaviour use the same number everywhere."""
        if self.world <= 1:
            return value
        import torch
        import torch.distributed as dist

        from verl_b200.single_controller.spmd import init_spmd_process_group

        t = torch.tensor([float(value)], dtype=torch.float64)
        dist.all_reduce(t, op={"min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX, "sum": dist.ReduceOp.SUM}[op], group=init_spmd_process_group())
        return float(t.item())

    def _switch_threshold(self) -> int:
        """Prompt groups that must be sampleable before the training GPUs are taken back (at least one mini-batch)."""
        mini = max(1, self.train_batch_size // self.parameter_sync_step)
        if self._controller is not None:
            # training cannot start on lent GPUs: a policy that would rather keep them lent still hands them back once the
            # whole batch is there
            need = self._controller.wait_threshold(self.global_steps, self._schedule_context(self.global_steps))
            return self.train_batch_size if need is None else min(need, self.train_batch_size)
        return min(max(round(self._switch_threshold_ratio * self.train_batch_size), mini), self.train_batch_size)

    def _sampleable(self, step: int) -> int:
        return int(self._agree(self.replay_buffer.get_sampleable_count(step, self.partition_id) * self.world, "min"))

    def switch_to_rollout(self):
        """Wake the colocated engine on the committed weights and let the balancer route requests to it."""
        t0 = time.perf_counter()
        self.stages.actor_rollout_wg.update_weights()
        self._hybrid_replica.wake_up()
        if getattr(self._hybrid_replica.server, "resume", None) is not None:
            self._hybrid_replica.server.resume()
        self._servers.add_server(self._hybrid_name, self._hybrid_replica.server)
        self.current_mode = HybridEngineMode.ROLLOUT
        self._to_rollout_costs.append(time.perf_counter() - t0)
        self.switch_log.append(("rollout", self.global_steps))

    def switch_to_trainer(self):
        """Stop routing to the colocated engine, hand its open requests to the pool (the clients resume them with the tokens
        generated so far) and release its KV cache for training."""
        t0 = time.perf_counter()
        self._servers.remove_server(self._hybrid_name)
        self._hybrid_replica.abort_all_requests()
        self._hybrid_replica.server.wait_idle(timeout=60.0)
        self._hybrid_replica.sleep()
        self.current_mode = HybridEngineMode.TRAINER
        self._to_trainer_costs.append(time.perf_counter() - t0)
        self.switch_log.append(("trainer", self.global_steps))

    def _adapt_switch_threshold(self, had_idle: bool) -> None:
        c = self.hybrid_rollout_config
        if had_idle:
            self._calm_steps = 0
            self._idle_steps = min(self._idle_steps + 1, c.switch_threshold_release_steps)
            if self._idle_steps >= c.switch_threshold_release_steps:
                self._switch_threshold_ratio = min(1.0, self._switch_threshold_ratio + c.switch_threshold_step_up)
            return
        self._idle_steps = 0
        self._calm_steps = min(self._calm_steps + 1, c.switch_threshold_release_steps)
        if self._calm_steps >= c.switch_threshold_release_steps:
            self._switch_threshold_ratio = max(1.0 / self.parameter_sync_step, self._switch_threshold_ratio - c.switch_threshold_step_down)

    def _effective_switch_cost(self):
        if not self._to_rollout_costs or not self._to_trainer_costs:
            return None
        return sum(self._to_rollout_costs) / len(self._to_rollout_costs) + sum(self._to_trainer_costs) / len(self._to_trainer_costs)

    def _lending_decision(self, total_steps: int) -> dict:
        """After a step: adapt the threshold, then lend the GPUs for the coming wait if that is expected to pay."""
        c = self.hybrid_rollout_config
        self._consumed_groups += self.train_batch_size
        if self._controller is not None:
            ctl = self._controller
            ctl.last_activate_duration_s = self._to_rollout_costs[-1] if self._to_rollout_costs else 0.0
            ctl.last_deactivate_duration_s = self._to_trainer_costs[-1] if self._to_trainer_costs else 0.0
            return ctl.after_weight_sync(self.global_steps, self._schedule_context(self.global_steps + 1), more_steps=self.global_steps < total_steps)
        poll = max(5.0 * float(getattr(self.replay_buffer, "poll_interval_s", 0.01)), 0.05)
        had_idle = self._agree(self._step_sample_wait_seconds, "max") > poll        # the step really waited for trajectories
        if self._step_wait_samples > 0 and self._step_sample_wait_seconds > 0:
            self._wait_seconds += self._step_sample_wait_seconds
            self._wait_samples += self._step_wait_samples
        ratio_used = self._switch_threshold_ratio
        if c.adaptive_switch_threshold:
            self._adapt_switch_threshold(had_idle)
        threshold = self._switch_threshold()
        sampleable = self._sampleable(self.global_steps + 1)
        remaining = max(0, threshold - sampleable)
        per_sample = self._agree(self._wait_seconds / self._wait_samples, "max") if self._wait_samples > 0 else None
        cost = self._effective_switch_cost()
        cost = self._agree(cost, "max") if cost is not None else None
        benefit = remaining * per_sample * (1.0 - 1.0 / self._scaling_factor) if per_sample is not None else None
        should = self.global_steps < total_steps and remaining > 0 and (benefit is None or cost is None or benefit > cost)
        m = {"separate_async/switch/threshold_ratio": ratio_used, "separate_async/switch/wait_samples": float(self._step_wait_samples),
             "separate_async/switch/idle": float(had_idle), "separate_async/decision/sampleable_count": float(sampleable),
             "separate_async/decision/remaining": float(remaining), "separate_async/decision/should_switch_to_rollout": float(should)}
        if per_sample is not None:
            m["separate_async/decision/per_sample_time_seconds"] = per_sample
        if cost is not None:
            m["separate_async/decision/effective_switch_cost_seconds"] = cost
        if should and self.current_mode == HybridEngineMode.TRAINER:
            self.switch_to_rollout()
        return m

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
        if not self._switch_enabled:
            return
        self._step_sample_wait_seconds = 0.0
        self._step_wait_samples = 0
        if self.current_mode == HybridEngineMode.ROLLOUT and self._sampleable(self.global_steps) >= self._switch_threshold():
            self._take_back()

    def on_sample_begin(self):
        need = max(1, self.train_batch_size // self.world)
        if self._switch_enabled:
            have = self.replay_buffer.get_sampleable_count(self.global_steps, self.partition_id)
            self._step_wait_samples += max(0, need - have)
            self._sample_start = time.perf_counter()
            if self.current_mode == HybridEngineMode.ROLLOUT:
                # the GPUs stay lent until enough of the batch exists; training cannot start before they are back
                self.replay_buffer.wait_for_sampleable(self.global_steps, self.partition_id, max(1, self._switch_threshold() // self.world))
                self._agree(0.0, "max")                # every rank has reached its share: switch together
                self._take_back()
        self.replay_buffer.wait_for_sampleable(self.global_steps, self.partition_id, need)

    def on_sample_end(self):
        if self._switch_enabled:
            self._step_sample_wait_seconds += time.perf_counter() - self._sample_start

    def step(self, metrics: dict, timing_raw: dict):
        out = super().step(metrics, timing_raw)
        metrics.update(self.sync_weights())
        if self._switch_enabled:
            metrics.update(self._lending_decision(int(self.stages.total_training_steps)))
        return out

    def on_validate_begin(self):
        if self._switch_enabled and self.current_mode == HybridEngineMode.ROLLOUT:
            self._take_back()               # validation generates on the colocated engine through the stage trainer

    def on_train_end(self):
        if self._switch_enabled and self.current_mode == HybridEngineMode.ROLLOUT:
            self._take_back()
        self.agent_loop.shutdown()
        for r in getattr(self, "_owned", []):
            r.shutdown()
        if self._export_file and os.path.exists(self._export_file):
            os.unlink(self._export_file)
