"""Asynchronous reward computation that overlaps with generation (reference: ``verl/experimental/reward_loop/
reward_loop.py:93-343`` — ``RewardLoopWorker`` CPU actors behind a ``RewardLoopManager``; optional reward-model servers).

A reward-loop manager scores ONE sample per call (``await run_single(sample)``), so the agent loop can score each
trajectory the moment it finishes. ``RewardLoopManager.compute_rm_score(batch)`` runs a whole batch through a pool of
worker threads and returns the ``rm_scores`` tensor (score at the last valid response token) plus extra infos.
"""

from __future__ import annotations

import asyncio
import concurrent.futures
from typing import Any, Callable, Optional

import numpy as np
import torch

from verl_b200.protocol import DataProto

__all__ = ["RewardLoopWorker", "RewardLoopManager", "get_reward_loop_manager_cls", "register_reward_loop"]

_REGISTRY: dict[str, type] = {}


def register_reward_loop(name: str):
    def deco(cls):
        _REGISTRY[name] = cls
        return cls

    return deco


def get_reward_loop_manager_cls(name: str):
    if name not in _REGISTRY:
        from . import reward_manager  # noqa: F401 - populate

    if name not in _REGISTRY:
        raise ValueError(f"unknown reward-loop manager {name!r}; known: {sorted(_REGISTRY)}")
    return _REGISTRY[name]


class RewardLoopWorker:
    """Holds one reward-loop manager instance; ``compute_score_batch`` scores rows concurrently on an event loop."""

    def __init__(self, config, tokenizer, compute_score: Optional[Callable] = None, manager_name: Optional[str] = None, rm_client=None):
        get = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
        rcfg = get("reward", None) or get("reward_model", None) or {}
        name = manager_name or (rcfg.get("reward_manager", "naive") if hasattr(rcfg, "get") else "naive")
        name = {"token_rule": "naive", "batch": "naive"}.get(name, name)
        self.manager = get_reward_loop_manager_cls(name)(config, tokenizer, compute_score, rm_client=rm_client)

    async def compute_score(self, sample: dict) -> dict:
        return await self.manager.run_single(sample)

    async def compute_score_batch(self, samples: list[dict]) -> list[dict]:
        return list(await asyncio.gather(*[self.manager.run_single(s) for s in samples]))


class RewardLoopManager:
    def __init__(self, config, tokenizer, compute_score: Optional[Callable] = None, num_workers: int = 4, manager_name: Optional[str] = None,
                 rm_client=None):
        self.tokenizer = tokenizer
        self.workers = [RewardLoopWorker(config, tokenizer, compute_score, manager_name, rm_client) for _ in range(max(1, num_workers))]
        self.pool = concurrent.futures.ThreadPoolExecutor(max_workers=len(self.workers), thread_name_prefix="reward-loop")

    @staticmethod
    def _samples(batch: DataProto) -> list[dict]:
        out = []
        for i in range(len(batch)):
            s = {k: v[i] for k, v in batch.non_tensor_batch.items()}
            n = int(batch.batch["attention_mask"][i, -batch.batch["responses"].shape[1]:].sum())
            s["response_ids"] = batch.batch["responses"][i, :n].tolist()
            s["valid_response_length"] = n
            out.append(s)
        return out

    def compute_rm_score(self, batch: DataProto) -> DataProto:
        samples = self._samples(batch)
        k = len(self.workers)
        chunks = [samples[i::k] for i in range(k)]
        futs = [self.pool.submit(lambda w=w, c=c: asyncio.run(w.compute_score_batch(c))) for w, c in zip(self.workers, chunks) if c]
        results: list[Any] = [None] * len(samples)
        for wi, f in enumerate(futs):
            for j, r in enumerate(f.result()):
                results[wi + j * k] = r
        R = batch.batch["responses"].shape[1]
        scores = torch.zeros(len(samples), R, dtype=torch.float32)
        extra: dict[str, list] = {}
        for i, (s, r) in enumerate(zip(samples, results)):
            n = s["valid_response_length"]
            if n > 0:
                scores[i, n - 1] = float(r["reward_score"])
            for kx, vx in (r.get("reward_extra_info") or {}).items():
                extra.setdefault(kx, [None] * len(samples))[i] = vx
        non_tensor = {k: np.array(v, dtype=object) for k, v in extra.items()}
        return DataProto.from_dict(tensors={"rm_scores": scores}, non_tensors=non_tensor)

    def shutdown(self):
        self.pool.shutdown(wait=False)
