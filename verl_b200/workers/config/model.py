"""Model section (``actor_rollout_ref.model`` / ``critic.model``). Reference: ``verl/workers/config/model.py:30-200``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from verl_b200.base_config import BaseConfig

from ._util import _sub, from_config  # noqa: F401

__all__ = ["HFModelConfig", "MtpConfig", "TiledMLPConfig"]


@dataclass
class MtpConfig(BaseConfig):
    """Multi-token prediction heads: trained alongside the policy and / or used as the draft of speculative decoding."""

    enable: bool = False
    enable_train: bool = False
    enable_rollout: bool = False
    detach_encoder: bool = False
    mtp_loss_scaling_factor: float = 0.1
    method: str = "mtp"
    num_speculative_tokens: int = 1
    speculative_algorithm: str = "EAGLE"
    speculative_num_steps: int = 3
    speculative_eagle_topk: int = 1
    speculative_num_draft_tokens: int = 4


@dataclass
class TiledMLPConfig(BaseConfig):
    """Run the MLP over ``num_shards`` slices of the token dimension, recomputing each slice in backward."""

    enabled: bool = False
    num_shards: int = 4


@dataclass
class HFModelConfig(BaseConfig):
    path: Any = None
    preset: Any = None
    hf_config_path: Any = None
    tokenizer_path: Any = None
    use_shm: bool = False
    trust_remote_code: bool = False
    custom_chat_template: Any = None
    external_lib: Any = None
    override_config: dict = field(default_factory=lambda: {})
    enable_gradient_checkpointing: bool = True
    enable_activation_offload: bool = False
    use_remove_padding: bool = True
    use_fused_kernels: bool = True
    fused_kernel_options: dict = field(default_factory=lambda: {'impl_backend': 'native'})
    use_liger: bool = False
    lora_rank: int = 0
    lora_alpha: int = 16
    target_modules: str = 'all-linear'
    exclude_modules: Any = None
    lora_adapter_path: Any = None
    lora: dict = field(default_factory=lambda: {'type': 'lora', 'merge': False, 'rank': 0, 'alpha': 32, 'dropout': 0.0, 'target_modules': ['linear_qkv', 'linear_proj', 'linear_fc1', 'linear_fc2'], 'exclude_modules': [], 'adapter_path': None, 'freeze_vision_model': True, 'freeze_vision_projection': True, 'freeze_language_model': True})
    tiled_mlp: TiledMLPConfig = _sub(TiledMLPConfig)
    mtp: MtpConfig = _sub(MtpConfig)
    value_head: bool = False
    _mutable_fields = {"path", "tokenizer_path", "hf_config_path"}

    def __post_init__(self):
        if self.lora_rank < 0:
            raise ValueError("model.lora_rank must be >= 0")
        if self.fused_kernel_options.get("impl_backend") not in (None, "native", "torch", "triton", "liger"):
            raise ValueError(f"unknown fused kernel backend {self.fused_kernel_options.get('impl_backend')!r}")

    @property
    def source(self) -> Optional[str]:
        return self.path or self.preset

    def validate(self):
        """A run needs weights from somewhere: a model directory or an architecture preset."""
        if not self.source:
            raise ValueError("model.path (a Hugging Face directory) or model.preset (a built-in architecture) must be set")
