"""Engine sections (``fsdp_config`` / ``megatron``). Reference: ``verl/workers/config/engine.py``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from verl_b200.base_config import BaseConfig

from ._util import _sub, from_config  # noqa: F401

__all__ = ["QATEngineConfig", "FSDPEngineConfig", "McoreEngineConfig", "RouterReplayConfig"]


@dataclass
class QATEngineConfig(BaseConfig):
    enable: bool = False
    mode: str = "w4a16"
    group_size: int = 16
    ignore_patterns: list = field(default_factory=lambda: ["lm_head", "embed_tokens", "re:.*mlp.gate$"])
    activation_observer: str = "static_minmax"
    quantization_config_path: Any = None


@dataclass
class RouterReplayConfig(BaseConfig):
    """``disabled`` | ``R2`` (the old-log-prob pass records the routing, the update replays it) | ``R3`` (the rollout records)."""

    mode: str = "disabled"
    record_file: Any = None
    replay_file: Any = None

    def __post_init__(self):
        if str(self.mode).upper() not in ("DISABLED", "R2", "R3"):
            raise ValueError(f"router_replay.mode must be disabled, R2 or R3, got {self.mode!r}")


@dataclass
class FSDPEngineConfig(BaseConfig):
    strategy: str = 'fsdp'
    fsdp_size: int = -1
    param_offload: bool = False
    optimizer_offload: bool = False
    offload_policy: bool = False
    reshard_after_forward: bool = False
    zero3: bool = False
    expert_parallel_size: int = 1
    ulysses_sequence_parallel_size: int = 1
    context_parallel_size: int = 1
    context_parallel_zigzag: bool = False
    dynamic_context_parallel: bool = False
    max_seqlen_per_dp_cp_rank: Optional[int] = None
    model_dtype: Any = None
    dtype: str = 'bfloat16'
    forward_prefetch: bool = False
    use_symmetric_memory: bool = True
    wrap_policy: dict = field(default_factory=lambda: {'min_num_params': 0})
    use_orig_params: bool = False
    seed: int = 0
    full_determinism: bool = False
    use_torch_compile: bool = False
    entropy_from_logits_with_chunking: bool = False
    entropy_from_logits_chunk_size: int = 2048
    entropy_checkpointing: bool = False
    use_no_sync_for_gradient_accumulation: bool = False
    pad_to_length: bool = False
    pad_to_length_bucket: int = 1024
    forward_only: bool = False
    qat: QATEngineConfig = _sub(QATEngineConfig)

    def __post_init__(self):
        if self.strategy not in ("fsdp", "fsdp2", "fsdp_zero3"):
            raise ValueError(f"unknown fsdp strategy {self.strategy!r}")
        if self.ulysses_sequence_parallel_size > 1 and self.context_parallel_size > 1:
            raise ValueError("Ulysses sequence parallelism and context parallelism share the token dimension: enable one of them")
        if (self.reshard_after_forward or self.zero3) and (self.ulysses_sequence_parallel_size > 1 or self.context_parallel_size > 1):
            raise ValueError("row-sharded projections (reshard_after_forward) do not combine with sequence / context parallelism")


@dataclass
class McoreEngineConfig(BaseConfig):
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Any = None
    context_parallel_size: int = 1
    context_parallel_zigzag: bool = False
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: Any = None
    sequence_parallel: bool = True
    use_distributed_optimizer: bool = True
    use_dist_checkpointing: bool = False
    dist_checkpointing_path: Any = None
    dist_ckpt_optim_fully_reshardable: bool = False
    distrib_optim_fully_reshardable_mem_efficient: bool = False
    param_offload: bool = False
    grad_offload: bool = False
    optimizer_offload: bool = False
    seed: int = 0
    full_determinism: bool = False
    dtype: str = 'bfloat16'
    use_mbridge: bool = True
    vanilla_mbridge: bool = True
    use_remove_padding: bool = True
    forward_only: bool = False
    dynamic_context_parallel: bool = False
    max_seqlen_per_dp_cp_rank: Any = None
    override_ddp_config: dict = field(default_factory=lambda: {})
    override_transformer_config: dict = field(default_factory=lambda: {'recompute_granularity': None, 'recompute_modules': ['core_attn'], 'recompute_method': None, 'recompute_num_layers': None, 'attention_backend': 'flash'})
    override_mcore_model_config: dict = field(default_factory=lambda: {})
    router_replay: RouterReplayConfig = _sub(RouterReplayConfig)

    def __post_init__(self):
        for k in ("tensor_model_parallel_size", "pipeline_model_parallel_size", "context_parallel_size", "expert_model_parallel_size"):
            if int(getattr(self, k)) < 1:
                raise ValueError(f"megatron.{k} must be >= 1")
        v = self.virtual_pipeline_model_parallel_size
        if v is not None and self.pipeline_model_parallel_size < 2 and int(v) > 1:
            raise ValueError("virtual pipeline stages need pipeline_model_parallel_size >= 2")

    @property
    def model_parallel_size(self) -> int:
        return self.tensor_model_parallel_size * self.pipeline_model_parallel_size * self.context_parallel_size
