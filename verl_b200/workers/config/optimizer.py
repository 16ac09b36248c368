"""Optimizer sections. Reference: ``verl/workers/config/optimizer.py``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from verl_b200.base_config import BaseConfig

from ._util import _sub, from_config  # noqa: F401

__all__ = ["OptimizerConfig", "FSDPOptimizerConfig", "McoreOptimizerConfig"]


@dataclass
class OptimizerConfig(BaseConfig):
    """Keys every engine's optimizer section has."""

    lr: float = 1e-6
    lr_warmup_steps_ratio: float = 0.0
    lr_warmup_steps: int = -1
    total_training_steps: int = -1
    weight_decay: float = 0.01
    betas: list = field(default_factory=lambda: [0.9, 0.999])
    eps: float = 1e-8
    clip_grad: float = 1.0
    lr_scheduler_type: str = "constant"
    min_lr_ratio: float = 0.0
    num_cycles: float = 0.5
    _mutable_fields = {"total_training_steps"}

    def __post_init__(self):
        if self.lr < 0:
            raise ValueError("optim.lr must be >= 0")
        if getattr(self, "warmup_style", None) is not None and self.lr_scheduler_type == "constant":
            object.__setattr__(self, "lr_scheduler_type", self.warmup_style)      # deprecated spelling
        if self.lr_scheduler_type not in ("constant", "cosine", "linear", "wsd", "inverse_square_root"):
            raise ValueError(f"unknown lr_scheduler_type {self.lr_scheduler_type!r}")

    def warmup_steps(self, total: Optional[int] = None) -> int:
        total = self.total_training_steps if total is None else total
        return self.lr_warmup_steps if self.lr_warmup_steps >= 0 else int(self.lr_warmup_steps_ratio * max(total, 0))


@dataclass
class FSDPOptimizerConfig(OptimizerConfig):
    optimizer: str = 'AdamW'
    optimizer_impl: str = 'verl_b200.fused_adamw'
    zero_indexed_step: bool = True
    warmup_style: Any = None
    override_optimizer_config: Any = None


@dataclass
class McoreOptimizerConfig(OptimizerConfig):
    optimizer: str = 'adam'
    lr_warmup_init: float = 0.0
    lr_decay_steps: Any = None
    lr_decay_style: str = 'constant'
    min_lr: float = 0.0
    weight_decay_incr_style: str = 'constant'
    lr_wsd_decay_style: str = 'exponential'
    lr_wsd_decay_steps: Any = None
    use_checkpoint_opt_param_scheduler: bool = False
    use_distributed_optimizer: bool = True
    override_optimizer_config: dict = field(default_factory=lambda: {})
