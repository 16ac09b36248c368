"""Critic section. Reference: ``verl/workers/config/critic.py``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from verl_b200.base_config import BaseConfig

from ._util import _sub, from_config  # noqa: F401
from verl_b200.trainer.config import CheckpointConfig

from .engine import FSDPEngineConfig, McoreEngineConfig
from .model import HFModelConfig
from .optimizer import FSDPOptimizerConfig, McoreOptimizerConfig, OptimizerConfig

__all__ = ["CriticConfig", "FSDPCriticConfig", "McoreCriticConfig"]


@dataclass
class CriticConfig(BaseConfig):
    rollout_n: Any = None
    strategy: str = 'fsdp'
    enable: Any = None
    ppo_mini_batch_size: Any = None
    ppo_micro_batch_size: Any = None
    ppo_micro_batch_size_per_gpu: Any = None
    use_dynamic_bsz: Any = None
    ppo_max_token_len_per_gpu: int = 32768
    forward_max_token_len_per_gpu: Any = None
    forward_micro_batch_size: Any = None
    forward_micro_batch_size_per_gpu: Any = None
    ppo_epochs: Any = None
    shuffle: Any = None
    data_loader_seed: int = 42
    cliprange_value: float = 0.5
    loss_agg_mode: Any = None
    loss_scale_factor: Any = None
    ulysses_sequence_parallel_size: int = 1
    grad_clip: float = 1.0
    nccl_timeout: int = 600
    optim: OptimizerConfig = _sub(OptimizerConfig)
    model: HFModelConfig = _sub(HFModelConfig)
    checkpoint: CheckpointConfig = _sub(CheckpointConfig)
    profiler: Any = None
    _mutable_fields = {"ppo_mini_batch_size", "ppo_micro_batch_size", "ppo_micro_batch_size_per_gpu", "rollout_n"}

    def __post_init__(self):
        assert self.strategy in ("fsdp", "fsdp2", "megatron"), f"unknown strategy {self.strategy}"
        if not self.use_dynamic_bsz and self.ppo_micro_batch_size is not None and self.ppo_micro_batch_size_per_gpu not in (None, self.ppo_micro_batch_size):
            raise ValueError("set either critic.ppo_micro_batch_size or critic.ppo_micro_batch_size_per_gpu, not both")
        if float(self.cliprange_value) < 0:
            raise ValueError("critic.cliprange_value must be >= 0")


@dataclass
class FSDPCriticConfig(CriticConfig):
    strategy: str = "fsdp"
    optim: FSDPOptimizerConfig = _sub(FSDPOptimizerConfig)
    fsdp_config: FSDPEngineConfig = _sub(FSDPEngineConfig)
    megatron: dict = field(default_factory=dict)


@dataclass
class McoreCriticConfig(CriticConfig):
    strategy: str = "megatron"
    load_weight: bool = True
    optim: McoreOptimizerConfig = _sub(McoreOptimizerConfig)
    megatron: McoreEngineConfig = _sub(McoreEngineConfig)
