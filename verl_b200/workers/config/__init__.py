"""Typed views of the yaml config sub-trees (reference: ``verl/workers/config/{model,actor,critic,rollout,engine,
optimizer,reward,distillation,disaggregation}.py``). Every class is a frozen, mapping-like dataclass: attribute and ``[]``
access both work, unknown yaml keys are ignored by ``from_config``, cross-field checks run in ``__post_init__``. The field
sets follow the group files under ``verl_b200/trainer/config`` (a test keeps the two in step)."""

from verl_b200.trainer.config import (AlgoConfig, CheckpointConfig, DataConfig, FilterGroupsConfig, HybridRolloutSwitchConfig, KLControlConfig,
                                      PFPPOConfig, RolloutCorrectionConfig, TrainerConfig)

from ._util import from_config
from .actor import ActorConfig, FSDPActorConfig, McoreActorConfig, PolicyLossConfig
from .critic import CriticConfig, FSDPCriticConfig, McoreCriticConfig
from .disaggregation import DisaggregationConfig
from .distillation import DistillationConfig, DistillationLossConfig
from .engine import FSDPEngineConfig, McoreEngineConfig, QATEngineConfig, RouterReplayConfig
from .model import HFModelConfig, MtpConfig, TiledMLPConfig
from .optimizer import FSDPOptimizerConfig, McoreOptimizerConfig, OptimizerConfig
from .reward import CustomRewardFunctionConfig, RewardConfig, RewardModelConfig, SandboxFusionConfig
from .rollout import (AgentLoopConfig, CheckpointEngineConfig, CustomAsyncServerConfig, MultiTurnConfig, PrometheusConfig, RolloutConfig, SamplingConfig,
                      TraceConfig)

__all__ = ["ActorConfig", "AgentLoopConfig", "AlgoConfig", "CheckpointConfig", "CheckpointEngineConfig", "CriticConfig", "CustomAsyncServerConfig",
           "CustomRewardFunctionConfig", "DataConfig", "DisaggregationConfig", "DistillationConfig", "DistillationLossConfig", "FSDPActorConfig",
           "FSDPCriticConfig", "FSDPEngineConfig", "FSDPOptimizerConfig", "FilterGroupsConfig", "HFModelConfig", "HybridRolloutSwitchConfig",
           "KLControlConfig", "McoreActorConfig", "McoreCriticConfig", "McoreEngineConfig", "McoreOptimizerConfig", "MtpConfig", "MultiTurnConfig",
           "OptimizerConfig", "PFPPOConfig", "PolicyLossConfig", "PrometheusConfig", "QATEngineConfig", "RewardConfig", "RewardModelConfig",
           "RolloutConfig", "RolloutCorrectionConfig", "RouterReplayConfig", "SamplingConfig", "SandboxFusionConfig", "TiledMLPConfig", "TraceConfig",
           "TrainerConfig", "from_config"]
