"""Rollout section. Reference: ``verl/workers/config/rollout.py``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from verl_b200.base_config import BaseConfig

from ._util import _sub, from_config  # noqa: F401
from .disaggregation import DisaggregationConfig
from .model import MtpConfig

__all__ = ["SamplingConfig", "MultiTurnConfig", "CustomAsyncServerConfig", "AgentLoopConfig", "CheckpointEngineConfig", "TraceConfig", "PrometheusConfig",
           "RolloutConfig"]

ROLLOUT_NAMES = ("native", "vllm", "sglang", "trtllm", "hf", "naive")


@dataclass
class SamplingConfig(BaseConfig):
    """Sampling parameters of validation generations."""

    top_k: int = -1
    top_p: float = 1.0
    temperature: int = 0
    n: int = 1
    do_sample: bool = False


@dataclass
class MultiTurnConfig(BaseConfig):
    """Multi-turn / tool-calling conversations driven by the agent loop."""

    enable: bool = False
    max_assistant_turns: Any = None
    max_user_turns: Any = None
    tool_config_path: Any = None
    function_tool_path: Any = None
    max_parallel_calls: int = 1
    max_tool_response_length: int = 256
    tool_response_truncate_side: str = 'middle'
    use_inference_chat_template: bool = False
    tokenization_sanity_check_mode: str = 'strict'
    format: str = 'hermes'
    num_repeat_rollouts: Any = None


@dataclass
class CustomAsyncServerConfig(BaseConfig):
    path: Any = None
    name: Any = None


@dataclass
class AgentLoopConfig(BaseConfig):
    num_workers: int = 8
    default_agent_loop: str = "single_turn_agent"
    agent_loop_config_path: Any = None
    client: str = "sync"
    custom_async_server: CustomAsyncServerConfig = _sub(CustomAsyncServerConfig)


@dataclass
class CheckpointEngineConfig(BaseConfig):
    """Actor -> rollout weight hand-off backend and its bucket size."""

    backend: str = 'naive'
    update_weights_bucket_megabytes: int = 2048
    engine_kwargs: dict = field(default_factory=lambda: {})
    custom_backend_module: Any = None


@dataclass
class TraceConfig(BaseConfig):
    """Per-request rollout traces."""

    project_name: Any = None
    experiment_name: Any = None
    backend: Any = None
    token2text: bool = False
    max_samples_per_step_per_worker: Any = None


@dataclass
class PrometheusConfig(BaseConfig):
    """Metrics endpoint of the rollout servers."""

    enable: bool = False
    port: int = 9090
    file: str = '/tmp/verl_b200/prometheus.yml'
    served_model_name: Any = None


@dataclass
class RolloutConfig(BaseConfig):
    name: str = 'native'
    mode: str = 'sync'
    nnodes: int = 0
    n_gpus_per_node: Any = None
    n: int = 1
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    do_sample: bool = True
    seed: int = 42
    full_determinism: bool = False
    prompt_length: Any = None
    response_length: Any = None
    dtype: str = 'bfloat16'
    gpu_memory_utilization: float = 0.5
    standalone_gpu_memory_utilization: Any = None
    ignore_eos: bool = False
    enforce_eager: bool = False
    cudagraph_capture_sizes: Any = None
    free_cache_engine: bool = True
    tensor_model_parallel_size: int = 1
    data_parallel_size: int = 1
    expert_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    max_num_batched_tokens: int = 8192
    max_model_len: Any = None
    max_num_seqs: int = 256
    enable_chunked_prefill: bool = True
    enable_prefix_caching: bool = True
    logprobs_mode: str = 'processed_logprobs'
    scheduling_policy: str = 'fcfs'
    load_format: str = 'dummy'
    layered_summon: bool = False
    disable_log_stats: bool = True
    log_stats: bool = False
    over_sample_rate: int = 0
    multi_stage_wake_up: bool = False
    calculate_log_probs: bool = True
    topk_log_probs: int = 0
    quantization: Any = None
    quantization_config_file: Any = None
    sync_interval: int = 16
    num_blocks: Any = None
    skip_tokenizer_init: bool = True
    enable_rollout_routing_replay: bool = False
    moe_load_balance_metrics_interval: int = 0
    log_prob_micro_batch_size: Any = None
    log_prob_micro_batch_size_per_gpu: Any = None
    log_prob_use_dynamic_bsz: Any = None
    log_prob_max_token_len_per_gpu: Any = None
    engine_kwargs: dict = field(default_factory=lambda: {'vllm': {}, 'sglang': {}, 'trtllm': {}, 'native': {}})
    router_config_path: Any = None
    skip: dict = field(default_factory=lambda: {'enable': False, 'dump_dir': '~/.verl_b200/rollout_dump', 'max_dump_step': 1})
    mtp: Any = None
    val_kwargs: SamplingConfig = _sub(SamplingConfig)
    multi_turn: MultiTurnConfig = _sub(MultiTurnConfig)
    agent: AgentLoopConfig = _sub(AgentLoopConfig)
    checkpoint_engine: CheckpointEngineConfig = _sub(CheckpointEngineConfig)
    trace: TraceConfig = _sub(TraceConfig)
    prometheus: PrometheusConfig = _sub(PrometheusConfig)
    disaggregation: DisaggregationConfig = _sub(DisaggregationConfig)
    profiler: Any = None
    _mutable_fields = {"max_model_len", "n"}

    def __post_init__(self):
        if self.name not in ROLLOUT_NAMES:
            raise ValueError(f"unknown rollout engine {self.name!r}; known: {ROLLOUT_NAMES}")
        if self.mode not in ("sync", "async"):
            raise ValueError(f"rollout.mode must be sync or async, got {self.mode!r}")
        if self.quantization not in (None, "fp8", "fp8_block"):
            raise ValueError(f"unsupported rollout.quantization {self.quantization!r}")
        if self.pipeline_model_parallel_size != 1:
            raise ValueError("rollout.pipeline_model_parallel_size > 1 is not supported by the in-house engine")
        if not 0.0 < float(self.gpu_memory_utilization) <= 1.0:
            raise ValueError("rollout.gpu_memory_utilization must be in (0, 1]")
        if self.checkpoint_engine.backend not in ("naive", "nccl", "delta_sharded", "peer"):
            raise ValueError(f"unknown checkpoint engine backend {self.checkpoint_engine.backend!r}")

    def replicas(self, world: int) -> int:
        per = self.tensor_model_parallel_size * self.data_parallel_size * self.pipeline_model_parallel_size
        assert world % per == 0, f"world size {world} is not a multiple of tp*dp*pp = {per}"
        return world // per
