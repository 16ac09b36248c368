"""Reward plumbing of the trainer: load the reward manager / custom score function, run it on a batch.

Parity target: ``verl/trainer/ppo/reward.py`` (get_custom_reward_fn :50, load_reward_manager :111, compute_reward :160).
"""

from __future__ import annotations

import importlib.util
import os
import sys
from functools import partial

from verl_b200.protocol import DataProto
from verl_b200.workers.reward_manager import get_reward_manager_cls

__all__ = ["get_custom_reward_fn", "load_reward_manager", "compute_reward", "extract_reward"]


def _g(cfg, key, default=None):
    cur = cfg
    for part in key.split("."):
        if cur is None:
            return default
        cur = cur.get(part) if hasattr(cur, "get") else getattr(cur, part, None)
    return default if cur is None else cur


def get_custom_reward_fn(config):
    """Load ``reward.custom_reward_function.{path,name}``; extra ``reward_kwargs`` are bound as keyword arguments."""
    path = _g(config, "reward.custom_reward_function.path") or _g(config, "custom_reward_function.path")
    if not path:
        return None
    if not os.path.exists(path):
        raise FileNotFoundError(f"Reward function file '{path}' not found.")
    name = _g(config, "reward.custom_reward_function.name") or _g(config, "custom_reward_function.name") or "compute_score"
    spec = importlib.util.spec_from_file_location("custom_module", path)
    module = importlib.util.module_from_spec(spec)
    try:
        sys.modules["custom_module"] = module
        spec.loader.exec_module(module)
    except Exception as e:
        raise RuntimeError(f"Error loading module from '{path}': {e}") from e
    if not hasattr(module, name):
        raise AttributeError(f"Reward function '{name}' not found in '{path}'.")
    fn = getattr(module, name)
    kwargs = dict(_g(config, "reward.reward_kwargs", {}) or {})
    return partial(fn, **kwargs) if kwargs else fn


def load_reward_manager(config, tokenizer, num_examine: int = 0, **reward_kwargs):
    name = _g(config, "reward.reward_manager") or _g(config, "reward_model.reward_manager") or "naive"
    cls = get_reward_manager_cls(name)
    compute_score = get_custom_reward_fn(config)
    url = _g(config, "reward.sandbox_fusion.url")
    if compute_score is None and url:
        # code test cases go to the configured sandbox service; one semaphore bounds the requests of all scoring threads
        # (reference: verl/trainer/ppo/reward.py, sandbox_fusion branch of load_reward_manager)
        import threading

        from verl_b200.utils.reward_score import default_compute_score

        compute_score = partial(default_compute_score, sandbox_fusion_url=url,
                                concurrent_semaphore=threading.Semaphore(int(_g(config, "reward.sandbox_fusion.max_concurrent", 64))),
                                memory_limit_mb=int(_g(config, "reward.sandbox_fusion.memory_limit_mb", 1024)))
    return cls(tokenizer=tokenizer, num_examine=num_examine, compute_score=compute_score,
               reward_fn_key=_g(config, "data.reward_fn_key", "data_source"), **reward_kwargs)


def compute_reward(data: DataProto, reward_fn):
    try:
        res = reward_fn(data, return_dict=True)
        return res["reward_tensor"], res.get("reward_extra_info", {})
    except TypeError:
        return reward_fn(data), {}


def extract_reward(batch: DataProto):
    """Rewards computed upstream (agent loop / reward workers) arrive as ``rm_scores``."""
    return batch.batch["rm_scores"], {k: v for k, v in batch.non_tensor_batch.items() if k.startswith("reward_extra/")}
