from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any, Optional

from verl_b200.base_config import BaseConfig

__all__ = ["from_config", "HFModelConfig", "OptimizerConfig", "FSDPEngineConfig", "McoreEngineConfig", "CheckpointConfig", "PolicyLossConfig",
           "ActorConfig", "FSDPActorConfig", "McoreActorConfig", "CriticConfig", "SamplingConfig", "MultiTurnConfig", "AgentLoopConfig",
           "RolloutConfig", "KLControlConfig", "RolloutCorrectionConfig", "AlgoConfig"]


def from_config(cls, node, **extra):
    """Build ``cls`` from a yaml node (dict-like), recursing into fields whose default is itself a config dataclass."""
    if node is None:
        return cls(**extra)
    if isinstance(node, cls):
        return node
    kw = {}
    for f in dataclasses.fields(cls):
        if f.name.startswith("_") or f.name not in node:
            continue
        v = node[f.name]
        sub = f.metadata.get("cls")
        if sub is not None and v is not None and not isinstance(v, sub):
            v = from_config(sub, v)
        elif hasattr(v, "items") and not dataclasses.is_dataclass(v):
            v = dict(v)
        kw[f.name] = v
    kw.update(extra)
    return cls(**kw)


def _sub(cls):
    return field(default_factory=cls, metadata={"cls": cls})


@dataclass
class HFModelConfig(BaseConfig):
    path: Optional[str] = None
    preset: Optional[str] = None
    tokenizer_path: Optional[str] = None
    override_config: dict = field(default_factory=dict)
    enable_gradient_checkpointing: bool = True
    enable_activation_offload: bool = False
    use_remove_padding: bool = True          # packed batches are the only layout of this framework
    use_fused_kernels: bool = True           # fused lm_head → log-prob kernels
    fused_kernel_options: dict = field(default_factory=lambda: {"impl_backend": "tcgen05"})
    trust_remote_code: bool = False
    lora_rank: int = 0
    lora_alpha: int = 16
    target_modules: Any = "all-linear"
    use_liger: bool = False
    use_shm: bool = False
    external_lib: Optional[str] = None

    def __post_init__(self):
        if self.path is None and self.preset is None:
            raise ValueError("model.path or model.preset must be set")
        if not self.use_remove_padding:
            raise ValueError("use_remove_padding=False is not available: batches are always packed")


@dataclass
class OptimizerConfig(BaseConfig):
    lr: float = 1e-6
    lr_warmup_steps_ratio: float = 0.0
    lr_warmup_steps: int = -1
    total_training_steps: int = -1
    weight_decay: float = 0.01
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    clip_grad: float = 1.0
    min_lr_ratio: float = 0.0
    num_cycles: float = 0.5
    lr_scheduler_type: str = "constant"
    optimizer: str = "AdamW"
    _mutable_fields = {"total_training_steps"}

    def __post_init__(self):
        assert self.lr >= 0 and self.lr_scheduler_type in ("constant", "cosine"), "lr must be ≥ 0 and scheduler constant|cosine"


@dataclass
class FSDPEngineConfig(BaseConfig):
    strategy: str = "fsdp"
    fsdp_size: int = -1
    param_offload: bool = False
    optimizer_offload: bool = False
    offload_policy: bool = False
    reshard_after_forward: bool = False      # False = resident bf16 parameters (ZeRO-2); True = gather per layer (ZeRO-3)
    expert_parallel_size: int = 1            # mixture-of-experts: 1 = every rank holds all experts; world size = experts spread over all ranks
    forward_prefetch: bool = False
    model_dtype: Optional[str] = None
    use_orig_params: bool = False
    ulysses_sequence_parallel_size: int = 1
    entropy_from_logits_with_chunking: bool = False
    use_torch_compile: bool = False          # accepted for compatibility; there is no tracing compiler in the hot path
    entropy_checkpointing: bool = False
    forward_only: bool = False
    use_symmetric_memory: bool = True
    seed: int = 0
    wrap_policy: dict = field(default_factory=dict)


@dataclass
class McoreEngineConfig(BaseConfig):
    strategy: str = "megatron"
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Optional[int] = None
    context_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: Optional[int] = None
    sequence_parallel: bool = True
    use_distributed_optimizer: bool = True
    param_offload: bool = False
    grad_offload: bool = False
    optimizer_offload: bool = False
    use_dist_checkpointing: bool = False
    model_dtype: Optional[str] = None
    forward_only: bool = False
    seed: int = 0
    override_transformer_config: dict = field(default_factory=dict)

    def __post_init__(self):
        for k in ("tensor_model_parallel_size", "pipeline_model_parallel_size", "context_parallel_size", "expert_model_parallel_size"):
            assert int(getattr(self, k)) >= 1, f"{k} must be ≥ 1"


@dataclass
class CheckpointConfig(BaseConfig):
    save_contents: list = field(default_factory=lambda: ["model", "optimizer", "extra"])
    load_contents: list = field(default_factory=lambda: ["model", "optimizer", "extra"])
    async_save: bool = False


@dataclass
class PolicyLossConfig(BaseConfig):
    loss_mode: str = "vanilla"
    clip_cov_ratio: float = 0.0002
    clip_cov_lb: float = 1.0
    clip_cov_ub: float = 5.0
    kl_cov_ratio: float = 0.0002
    ppo_kl_coef: float = 0.1
    rollout_correction: dict = field(default_factory=dict)


@dataclass
class ActorConfig(BaseConfig):
    strategy: str = "fsdp"
    ppo_mini_batch_size: int = 256
    ppo_micro_batch_size: Optional[int] = None
    ppo_micro_batch_size_per_gpu: Optional[int] = None
    use_dynamic_bsz: bool = False
    ppo_max_token_len_per_gpu: int = 16384
    use_prefix_grouper: bool = False     # share one prompt forward/backward among the n responses of its group
    clip_ratio: float = 0.2
    clip_ratio_low: float = 0.2
    clip_ratio_high: float = 0.2
    clip_ratio_c: float = 3.0
    loss_agg_mode: str = "token-mean"
    loss_scale_factor: Optional[int] = None
    entropy_coeff: float = 0.0
    calculate_entropy: bool = False
    use_kl_loss: bool = False
    kl_loss_coef: float = 0.001
    kl_loss_type: str = "low_var_kl"
    ppo_epochs: int = 1
    shuffle: bool = False
    data_loader_seed: int = 42
    use_torch_compile: bool = False
    policy_loss: PolicyLossConfig = _sub(PolicyLossConfig)
    optim: OptimizerConfig = _sub(OptimizerConfig)
    checkpoint: CheckpointConfig = _sub(CheckpointConfig)
    _mutable_fields = {"ppo_mini_batch_size", "ppo_micro_batch_size", "ppo_micro_batch_size_per_gpu"}

    def __post_init__(self):
        assert self.strategy in ("fsdp", "fsdp2", "megatron"), f"unknown strategy {self.strategy}"
        if not self.use_dynamic_bsz:
            if self.ppo_micro_batch_size is not None and self.ppo_micro_batch_size_per_gpu is not None:
                raise ValueError("set either actor.ppo_micro_batch_size or actor.ppo_micro_batch_size_per_gpu, not both "
                                 "(the former is deprecated)")
        assert self.loss_agg_mode in ("token-mean", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm"), self.loss_agg_mode

    def validate(self, n_gpus: int, train_batch_size: int, model_parallel: int = 1):
        """Batch-size arithmetic of the reference: the mini batch must divide the train batch, and the per-GPU micro
        batch must divide the per-GPU mini batch."""
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
    grad_clip: float = 1.0
    ulysses_sequence_parallel_size: int = 1
    entropy_from_logits_with_chunking: bool = False
    entropy_checkpointing: bool = False
    fsdp_config: FSDPEngineConfig = _sub(FSDPEngineConfig)


@dataclass
class McoreActorConfig(ActorConfig):
    strategy: str = "megatron"
    data_loader_seed: int = 42
    load_weight: bool = True
    megatron: McoreEngineConfig = _sub(McoreEngineConfig)


@dataclass
class CriticConfig(BaseConfig):
    strategy: str = "fsdp"
    enable: Optional[bool] = None
    ppo_mini_batch_size: int = 256
    ppo_micro_batch_size_per_gpu: Optional[int] = None
    use_dynamic_bsz: bool = False
    ppo_max_token_len_per_gpu: int = 32768
    forward_max_token_len_per_gpu: int = 32768
    ppo_epochs: int = 1
    shuffle: bool = False
    cliprange_value: float = 0.5
    loss_agg_mode: str = "token-mean"
    optim: OptimizerConfig = _sub(OptimizerConfig)
    checkpoint: CheckpointConfig = _sub(CheckpointConfig)


@dataclass
class SamplingConfig(BaseConfig):
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    do_sample: bool = True
    n: int = 1


@dataclass
class MultiTurnConfig(BaseConfig):
    enable: bool = False
    max_assistant_turns: Optional[int] = None
    max_user_turns: Optional[int] = None
    max_parallel_calls: int = 1
    max_tool_response_length: int = 256
    tool_response_truncate_side: str = "middle"
    tool_config_path: Optional[str] = None
    interaction_config_path: Optional[str] = None
    format: str = "hermes"

    def __post_init__(self):
        assert self.tool_response_truncate_side in ("left", "middle", "right")


@dataclass
class AgentLoopConfig(BaseConfig):
    num_workers: int = 8
    default_agent_loop: str = "single_turn_agent"
    agent_loop_config_path: Optional[str] = None
    client: str = "sync"


@dataclass
class RolloutConfig(BaseConfig):
    name: str = "native"
    mode: str = "sync"
    n: int = 1
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    do_sample: bool = True
    prompt_length: int = 512
    response_length: int = 512
    dtype: str = "bfloat16"
    gpu_memory_utilization: float = 0.5
    ignore_eos: bool = False
    enforce_eager: bool = False
    free_cache_engine: bool = True
    tensor_model_parallel_size: int = 1
    data_parallel_size: int = 1
    expert_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    max_num_batched_tokens: int = 8192
    max_model_len: Optional[int] = None
    max_num_seqs: int = 256
    enable_chunked_prefill: bool = True
    enable_prefix_caching: bool = True
    calculate_log_probs: bool = True
    topk_log_probs: int = 0      # return the sampler's k most likely tokens per step (needed by score centering)
    quantization: Optional[str] = None
    sync_interval: int = 16
    log_prob_micro_batch_size_per_gpu: Optional[int] = None
    log_prob_use_dynamic_bsz: bool = False
    log_prob_max_token_len_per_gpu: int = 16384
    enable_rollout_routing_replay: bool = False
    val_kwargs: SamplingConfig = field(default_factory=lambda: SamplingConfig(temperature=0.0, do_sample=False), metadata={"cls": SamplingConfig})
    multi_turn: MultiTurnConfig = _sub(MultiTurnConfig)
    agent: AgentLoopConfig = _sub(AgentLoopConfig)
    checkpoint_engine: dict = field(default_factory=lambda: {"backend": "naive", "update_weights_bucket_megabytes": 2048})

    def __post_init__(self):
        assert self.mode in ("sync", "async"), "rollout.mode must be sync or async"
        assert 0 < self.gpu_memory_utilization <= 1
        if self.quantization not in (None, "fp8"):
            raise ValueError(f"rollout.quantization={self.quantization!r}: only fp8 (128x128 block-scaled weights) is available")
        if self.pipeline_model_parallel_size != 1:
            raise NotImplementedError("rollout pipeline parallelism is not available")


@dataclass
class KLControlConfig(BaseConfig):
    type: str = "fixed"
    kl_coef: float = 0.001
    horizon: int = 10000
    target_kl: float = 0.1


@dataclass
class RolloutCorrectionConfig(BaseConfig):
    rollout_is: Optional[str] = None
    rollout_is_threshold: Any = 2.0
    rollout_is_batch_normalize: bool = False
    rollout_rs: Optional[str] = None
    rollout_rs_threshold: Any = None
    bypass_mode: bool = False
    loss_type: str = "ppo_clip"
    score_centering: bool = False

    def __post_init__(self):
        assert self.rollout_is in (None, "token", "sequence", "geometric"), self.rollout_is


@dataclass
class AlgoConfig(BaseConfig):
    gamma: float = 1.0
    lam: float = 1.0
    adv_estimator: str = "gae"
    norm_adv_by_std_in_grpo: bool = True
    use_kl_in_reward: bool = False
    kl_penalty: str = "kl"
    kl_ctrl: KLControlConfig = _sub(KLControlConfig)
    use_pf_ppo: bool = False
    pf_ppo: dict = field(default_factory=dict)
    filter_groups: dict = field(default_factory=dict)
    rollout_correction: Optional[RolloutCorrectionConfig] = field(default=None, metadata={"cls": RolloutCorrectionConfig})
