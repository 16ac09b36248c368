"""Actor / reference sections. Reference: ``verl/workers/config/actor.py``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from verl_b200.base_config import BaseConfig

from ._util import _sub, from_config  # noqa: F401
from verl_b200.trainer.config import CheckpointConfig
from verl_b200.utils.profiler.config import ProfilerConfig

from .engine import FSDPEngineConfig, McoreEngineConfig, QATEngineConfig, RouterReplayConfig
from .optimizer import FSDPOptimizerConfig, McoreOptimizerConfig, OptimizerConfig

__all__ = ["PolicyLossConfig", "ActorConfig", "FSDPActorConfig", "McoreActorConfig"]

LOSS_AGG_MODES = ("token-mean", "token-sum", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm")


@dataclass
class PolicyLossConfig(BaseConfig):
    loss_mode: str = "vanilla"
    clip_cov_ratio: float = 0.0002
    clip_cov_lb: float = 1.0
    clip_cov_ub: float = 5.0
    kl_cov_ratio: float = 0.0002
    ppo_kl_coef: float = 0.1
    dro_beta: Any = None


@dataclass
class ActorConfig(BaseConfig):
    rollout_n: Any = None
    strategy: str = 'fsdp'
    ppo_mini_batch_size: int = 256
    ppo_micro_batch_size: Any = None
    ppo_micro_batch_size_per_gpu: Any = None
    use_dynamic_bsz: bool = False
    ppo_max_token_len_per_gpu: int = 16384
    use_prefix_grouper: bool = False
    clip_ratio: float = 0.2
    clip_ratio_low: float = 0.2
    clip_ratio_high: float = 0.2
    clip_ratio_c: float = 3.0
    tau_pos: float = 1.0
    tau_neg: float = 1.05
    freeze_vision_tower: bool = False
    loss_agg_mode: str = 'token-mean'
    loss_scale_factor: Any = None
    entropy_coeff: float = 0.0
    calculate_entropy: bool = False
    calculate_sum_pi_squared: bool = False
    use_kl_loss: bool = False
    kl_loss_coef: float = 0.001
    kl_loss_type: str = 'low_var_kl'
    ppo_epochs: int = 1
    shuffle: bool = False
    data_loader_seed: int = 42
    use_torch_compile: bool = False
    use_fused_kernels: Any = None
    use_remove_padding: Any = None
    grad_clip: float = 1.0
    ulysses_sequence_parallel_size: int = 1
    entropy_from_logits_with_chunking: bool = False
    entropy_from_logits_chunk_size: int = 2048
    entropy_checkpointing: bool = False
    pad_to_length: bool = False
    policy_loss: PolicyLossConfig = _sub(PolicyLossConfig)
    optim: OptimizerConfig = _sub(OptimizerConfig)
    checkpoint: CheckpointConfig = _sub(CheckpointConfig)
    router_replay: RouterReplayConfig = _sub(RouterReplayConfig)
    qat: QATEngineConfig = _sub(QATEngineConfig)
    profiler: Any = None
    _mutable_fields = {"ppo_mini_batch_size", "ppo_micro_batch_size", "ppo_micro_batch_size_per_gpu", "rollout_n"}

    def __post_init__(self):
        assert self.strategy in ("fsdp", "fsdp2", "fsdp_zero3", "megatron"), f"unknown strategy {self.strategy}"
        if not self.use_dynamic_bsz:
            if self.ppo_micro_batch_size is not None and self.ppo_micro_batch_size_per_gpu is not None:
                raise ValueError("set either actor.ppo_micro_batch_size or actor.ppo_micro_batch_size_per_gpu, not both "
                                 "(the former is deprecated)")
        assert self.loss_agg_mode in LOSS_AGG_MODES, self.loss_agg_mode
        if not (0.0 <= float(self.clip_ratio_low) and 0.0 <= float(self.clip_ratio_high)):
            raise ValueError("clip ratios must be non-negative")

    def validate(self, n_gpus: int, train_batch_size: int, model_parallel: int = 1):
        """Batch-size arithmetic of the reference: the mini batch (counted in prompts) must not exceed the train batch, and the
        per-GPU micro batch must divide the per-GPU mini batch."""
        if self.use_dynamic_bsz:
            return
        if train_batch_size < self.ppo_mini_batch_size:
            raise ValueError(f"train_batch_size ({train_batch_size}) must be ≥ actor.ppo_mini_batch_size ({self.ppo_mini_batch_size})")
        if self.ppo_micro_batch_size_per_gpu is not None:
            dp = max(1, n_gpus // model_parallel)
            per_gpu = self.ppo_mini_batch_size // dp
            if per_gpu and per_gpu % self.ppo_micro_batch_size_per_gpu not in (0, per_gpu):
                raise ValueError(f"per-GPU mini batch {per_gpu} is not a multiple of ppo_micro_batch_size_per_gpu {self.ppo_micro_batch_size_per_gpu}")


@dataclass
class FSDPActorConfig(ActorConfig):
    strategy: str = "fsdp"
    optim: FSDPOptimizerConfig = _sub(FSDPOptimizerConfig)
    fsdp_config: FSDPEngineConfig = _sub(FSDPEngineConfig)
    megatron: dict = field(default_factory=dict)
    # reference-policy flavour of the same section
    log_prob_micro_batch_size: Any = None
    log_prob_micro_batch_size_per_gpu: Any = None
    log_prob_use_dynamic_bsz: bool = False
    log_prob_max_token_len_per_gpu: int = 16384


@dataclass
class McoreActorConfig(ActorConfig):
    strategy: str = "megatron"
    load_weight: bool = True
    optim: McoreOptimizerConfig = _sub(McoreOptimizerConfig)
    megatron: McoreEngineConfig = _sub(McoreEngineConfig)
    log_prob_micro_batch_size: Any = None
    log_prob_micro_batch_size_per_gpu: Any = None
    log_prob_use_dynamic_bsz: bool = False
    log_prob_max_token_len_per_gpu: int = 16384
