"""Replay buffers over TransferQueue tags (reference: ``verl/trainer/ppo/v1/replay_buffer.py:64-640``).

Every trajectory is one key of a partition with tags ``{uid, status ∈ pending|running|finished|failure, gen_step,
score}``. A prompt group (same ``uid``) becomes sampleable when all of its trajectories are terminal. ``sample`` draws
whole groups, evicts failed ones, optionally applies DAPO's group filter (drop groups whose scores are all equal), and —
in the async variant — drops groups generated more than ``max_off_policy_threshold`` steps ago.
"""

from __future__ import annotations

import time
from collections import Counter, defaultdict
from typing import Optional

from verl_b200.utils.transfer_queue import KVBatchMeta, TransferQueue, get_transfer_queue

__all__ = ["ReplayBuffer", "ReplayBufferAsync"]

TERMINAL = ("finished", "failure")


class ReplayBuffer:
    def __init__(self, tq: Optional[TransferQueue] = None, rollout_n: int = 1, filter_groups: bool = False, filter_metric: str = "score",
                 poll_interval_s: float = 0.01, timeout_s: float = 3600.0, max_off_policy_threshold: Optional[int] = None):
        self.tq = tq or get_transfer_queue()
        self.rollout_n, self.filter_groups, self.filter_metric = rollout_n, filter_groups, filter_metric
        self.poll_interval_s, self.timeout_s = poll_interval_s, timeout_s
        self.max_off_policy_threshold = max_off_policy_threshold
        self._validate_mode_config()

    def _validate_mode_config(self):
        assert self.max_off_policy_threshold is None, "the synchronous buffer trains on fresh samples only"

    # ------------------------------------------------------------------ group bookkeeping
    def _groups(self, partition_id: str) -> dict[str, list[tuple[str, dict]]]:
        groups: dict[str, list] = defaultdict(list)
        for key, tags in self.tq.kv_tags(partition_id).items():
            groups[tags.get("uid", key)].append((key, tags))
        return groups

    def _stale(self, tags: dict, global_steps: int) -> bool:
        return False

    def _classify(self, partition_id: str, global_steps: int):
        """→ (ready groups {uid: keys}, evictions Counter, keys to drop)."""
        ready, evict, drop = {}, Counter(), []
        for uid, members in self._groups(partition_id).items():
            if len(members) < self.rollout_n or not all(t.get("status") in TERMINAL for _, t in members):
                continue
            keys = [k for k, _ in members]
            if any(t.get("status") == "failure" for _, t in members):
                evict["failure"] += 1
                drop += keys
            elif any(self._stale(t, global_steps) for _, t in members):
                evict["stale"] += 1
                drop += keys
            elif self.filter_groups and len({t.get(self.filter_metric) for _, t in members}) <= 1:
                evict["filtered"] += 1
                drop += keys
            else:
                ready[uid] = sorted(keys)
        return ready, evict, drop

    def get_sampleable_count(self, global_steps: int, partition_id: str) -> int:
        return len(self._classify(partition_id, global_steps)[0])

    # ------------------------------------------------------------------ sampling
    def sample(self, global_steps: int, partition_id: str, batch_size: int) -> tuple[KVBatchMeta, dict]:
        """Blocks until ``batch_size`` prompt groups are ready; returns their trajectories (grouped, ``rollout_n`` each)."""
        t0 = time.time()
        evicted = Counter()
        while True:
            ready, ev, drop = self._classify(partition_id, global_steps)
            if drop:
                self.tq.kv_clear(partition_id, drop)
                evicted.update(ev)
            if len(ready) >= batch_size:
                break
            if time.time() - t0 > self.timeout_s:
                raise TimeoutError(f"replay buffer: {len(ready)}/{batch_size} prompt groups ready after {self.timeout_s}s")
            self.tq.wait(lambda: False, self.poll_interval_s)
        tags = self.tq.kv_tags(partition_id)
        order = sorted(ready, key=lambda u: (min(tags[k].get("gen_step", 0) for k in ready[u]), u))[:batch_size]   # oldest first
        keys = [k for u in order for k in ready[u]]
        stale = [global_steps - tags[k].get("gen_step", global_steps) for k in keys]
        metrics = {"replay/wait_s": time.time() - t0, "replay/ready_groups": len(ready), "replay/staleness_mean": sum(stale) / max(1, len(stale)),
                   "replay/staleness_max": max(stale, default=0), **{f"replay/evicted_{k}": v for k, v in evicted.items()}}
        return KVBatchMeta(partition_id, keys), metrics

    def release(self, meta: KVBatchMeta):
        self.tq.kv_clear(meta.partition_id, meta.keys)


class ReplayBufferAsync(ReplayBuffer):
    """Off-policy tolerant: groups older than ``max_off_policy_threshold`` steps are evicted instead of trained on."""

    def _validate_mode_config(self):
        assert self.max_off_policy_threshold is not None and self.max_off_policy_threshold >= 0

    def _stale(self, tags: dict, global_steps: int) -> bool:
        return global_steps - int(tags.get("gen_step", global_steps)) > self.max_off_policy_threshold

    def wait_for_sampleable(self, global_steps: int, partition_id: str, target_count: int, timeout_s: Optional[float] = None) -> int:
        t0 = time.time()
        while True:
            n = self.get_sampleable_count(global_steps, partition_id)
            if n >= target_count or time.time() - t0 > (timeout_s if timeout_s is not None else self.timeout_s):
                return n
            self.tq.wait(lambda: False, self.poll_interval_s)
