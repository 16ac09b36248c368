"""Reward-model serving for the reward loop: N replicas of the inference engine that hold the judge / reward model, one router
address in front of them, sleep / wake_up so that a colocated reward model gives its GPU memory back between scoring phases.

Reference: ``verl/experimental/reward_loop/reward_model.py:27-125`` (``RewardModelManager``: rollout replicas built from
``reward.reward_model.rollout``, colocated on a resource pool or standalone, a router process in front). Here a replica is
either an engine living in this process (colocated: it is handed in, e.g. built by a worker on its GPU) or a child process
started with ``python -m verl_b200.workers.rollout.replica`` (standalone); both speak the same HTTP endpoints to the router.
"""

from __future__ import annotations

from typing import Optional, Sequence

from verl_b200.workers.rollout.replica import RolloutMode, RolloutReplica

from .router import RouterClient, launch_router

__all__ = ["RewardModelManager"]


def _get(cfg, key, default=None):
    cur = cfg
    for part in key.split("."):
        if cur is None:
            return default
        cur = cur.get(part, None) if hasattr(cur, "get") else getattr(cur, part, None)
    return default if cur is None else cur


class RewardModelManager:
    """``config``: the ``reward.reward_model`` sub-tree (``model_path``, ``n_gpus_per_node``, ``nnodes``,
    ``rollout.{tensor_model_parallel_size, data_parallel_size, pipeline_model_parallel_size, free_cache_engine, max_num_seqs,
    max_model_len}``). ``engines``: already built engines to serve in-process (colocated mode); without them
    ``world_size // rollout_world_size`` standalone replica processes are started, one per GPU group."""

    def __init__(self, config, engines: Optional[Sequence] = None, tokenizer=None, eos_token_id=None, devices: Optional[Sequence[int]] = None):
        self.config = config
        self.tokenizer = tokenizer
        self.rollout_replicas: list[RolloutReplica] = []
        ro = _get(config, "rollout", {}) or {}
        self.rollout_world_size = (int(_get(ro, "tensor_model_parallel_size", 1)) * int(_get(ro, "data_parallel_size", 1))
                                   * int(_get(ro, "pipeline_model_parallel_size", 1)))
        if engines:
            for i, eng in enumerate(engines):
                rep = RolloutReplica(i, ro, mode=RolloutMode.COLOCATED)
                rep.init_hybrid(eng, eos_token_id=eos_token_id, tokenizer=tokenizer, http=True)
                self.rollout_replicas.append(rep)
        else:
            world = int(_get(config, "n_gpus_per_node", 1)) * int(_get(config, "nnodes", 1))
            n = world // self.rollout_world_size
            if n <= 0:
                raise ValueError(f"Not enough GPUs to run the reward model: world_size ({world}) < rollout_world_size ({self.rollout_world_size}). "
                                 "Check reward.reward_model.n_gpus_per_node / nnodes.")
            model = _get(config, "model_path", None) or _get(config, "model.path", None)
            if not model:
                raise ValueError("reward.reward_model.model_path is required for standalone reward-model replicas")
            extra = ["--max-num-seqs", str(int(_get(ro, "max_num_seqs", 256))), "--max-model-len", str(int(_get(ro, "max_model_len", 2048)))]
            for i in range(n):
                dev = devices[i] if devices is not None else i * self.rollout_world_size
                self.rollout_replicas.append(RolloutReplica(i, ro).init_standalone(model, device=dev, extra_args=extra))
        self.server_addresses = [r.address for r in self.rollout_replicas]
        self.router_address, self.router, self._stop_router = launch_router(self.server_addresses)
        if bool(_get(ro, "free_cache_engine", False)):
            self.sleep()

    def get_router_address(self) -> str:
        return self.router_address

    def client(self) -> RouterClient:
        """An ``rm_client`` for the reward-loop managers (``generate`` through the router)."""
        return RouterClient(self.router_address)

    def wake_up(self):
        for r in self.rollout_replicas:
            r.wake_up()

    def sleep(self):
        for r in self.rollout_replicas:
            r.sleep()

    def shutdown(self):
        self._stop_router()
        for r in self.rollout_replicas:
            r.shutdown()
