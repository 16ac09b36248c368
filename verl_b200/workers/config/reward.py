"""Reward section. Reference: ``verl/workers/config/reward.py``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from verl_b200.base_config import BaseConfig

from ._util import _sub, from_config  # noqa: F401

__all__ = ["CustomRewardFunctionConfig", "SandboxFusionConfig", "RewardModelConfig", "RewardConfig"]


@dataclass
class CustomRewardFunctionConfig(BaseConfig):
    path: Any = None
    name: str = "compute_score"


@dataclass
class SandboxFusionConfig(BaseConfig):
    url: Any = None
    max_concurrent: int = 64
    memory_limit_mb: int = 1024


@dataclass
class RewardModelConfig(BaseConfig):
    """Model-based reward: a scalar-head scorer on a training engine, or a generative judge behind a rollout replica."""

    enable: bool = False
    enable_resource_pool: bool = False
    n_gpus_per_node: int = 8
    nnodes: int = 0
    path: Any = None
    model_path: Any = None
    preset: Any = None
    strategy: str = 'fsdp'
    micro_batch_size_per_gpu: Any = None
    use_dynamic_bsz: bool = False
    forward_max_token_len_per_gpu: Any = None
    add_rule_reward: bool = True
    generative: bool = False
    judge_prompt_template: Any = None
    fsdp_config: dict = field(default_factory=lambda: {})
    rollout: dict = field(default_factory=lambda: {'name': 'native', 'dtype': 'bfloat16', 'gpu_memory_utilization': 0.5, 'tensor_model_parallel_size': 1, 'max_num_seqs': 1024, 'max_model_len': None, 'prompt_length': 2048, 'response_length': 2048, 'temperature': 1.0, 'top_p': 1.0, 'top_k': -1, 'do_sample': True, 'n': 1})


@dataclass
class RewardConfig(BaseConfig):
    num_workers: int = 8
    reward_manager: str = 'naive'
    reward_kwargs: dict = field(default_factory=lambda: {})
    custom_reward_function: CustomRewardFunctionConfig = _sub(CustomRewardFunctionConfig)
    reward_model: RewardModelConfig = _sub(RewardModelConfig)
    sandbox_fusion: SandboxFusionConfig = _sub(SandboxFusionConfig)

    @property
    def manager_name(self) -> str:
        """``reward_manager`` is a registered name, or the mapping form ``{source, name, module}`` of the reference."""
        rm = self.reward_manager
        return rm if isinstance(rm, str) else str((rm or {}).get("name", "naive"))
