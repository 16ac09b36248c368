"""On-policy distillation section. Reference: ``verl/workers/config/distillation.py``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from verl_b200.base_config import BaseConfig

from ._util import _sub, from_config  # noqa: F401

__all__ = ["DistillationLossConfig", "DistillationConfig"]


@dataclass
class DistillationLossConfig(BaseConfig):
    loss_mode: str = "k3"
    topk: int = 32
    use_task_rewards: bool = True
    distillation_loss_coef: float = 1.0
    loss_max_clamp: Any = None
    log_prob_min_clamp: Any = None
    use_policy_gradient: bool = False
    policy_loss_mode: str = "vanilla"
    clip_ratio: float = 0.2
    clip_ratio_low: float = 0.2
    clip_ratio_high: float = 0.2


@dataclass
class DistillationConfig(BaseConfig):
    enabled: bool = False
    enable: Any = None
    teacher_model: dict = field(default_factory=lambda: {'path': None, 'preset': None, 'override_config': {}, 'enable_gradient_checkpointing': False})
    topk: int = 32
    loss: str = 'forward_kl'
    jsd_beta: float = 0.5
    loss_coef: float = 1.0
    use_policy_loss: bool = False
    n_gpus_per_node: int = 8
    nnodes: int = 0
    teacher_key: str = 'data_source'
    teacher_models: dict = field(default_factory=lambda: {})
    teacher_mode: str = 'colocated'
    teacher_devices: Any = None
    teacher_addresses: dict = field(default_factory=lambda: {})
    distillation_loss: DistillationLossConfig = _sub(DistillationLossConfig)

    def __post_init__(self):
        if self.loss not in ("forward_kl", "reverse_kl", "jsd"):
            raise ValueError(f"unknown distillation loss {self.loss!r}")
        if self.teacher_mode not in ("colocated", "server"):
            raise ValueError(f"distillation.teacher_mode must be colocated or server, got {self.teacher_mode!r}")
        if int(self.topk) < 1:
            raise ValueError("distillation.topk must be >= 1")
