"""Prefill / decode disaggregation of rollout replicas. Reference: ``verl/workers/config/disaggregation.py:26``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from verl_b200.base_config import BaseConfig

from ._util import _sub, from_config  # noqa: F401

__all__ = ["DisaggregationConfig"]


@dataclass
class DisaggregationConfig(BaseConfig):
    """Separate prefill and decode replica pools; KV blocks travel over ``transfer_backend`` (NVLink peer copies here)."""

    enabled: bool = False
    prefill_replicas: int = 1
    decode_replicas: int = 1
    decode_tensor_model_parallel_size: Any = None
    transfer_backend: str = 'nvlink'
    bootstrap_port: Any = None
    ib_device: Any = None


    def __post_init__(self):
        if self.enabled and (int(self.prefill_replicas) < 1 or int(self.decode_replicas) < 1):
            raise ValueError("disaggregation needs at least one prefill and one decode replica")
