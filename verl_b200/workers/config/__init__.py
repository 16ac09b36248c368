"""Typed views of the yaml config sub-trees (reference: ``verl/workers/config/{model,actor,critic,rollout,engine,
optimizer}.py`` and ``verl/trainer/config/algorithm.py``). Every class is a frozen, mapping-like dataclass: attribute and
``[]`` access both work, unknown yaml keys are ignored by ``from_config``, cross-field checks run in ``__post_init__``."""

from .configs import (ActorConfig, AgentLoopConfig, AlgoConfig, CheckpointConfig, CriticConfig, FSDPActorConfig, FSDPEngineConfig, HFModelConfig,
                      KLControlConfig, McoreActorConfig, McoreEngineConfig, MultiTurnConfig, OptimizerConfig, PolicyLossConfig, RolloutConfig,
                      RolloutCorrectionConfig, SamplingConfig, from_config)

__all__ = ["ActorConfig", "AgentLoopConfig", "AlgoConfig", "CheckpointConfig", "CriticConfig", "FSDPActorConfig", "FSDPEngineConfig",
           "HFModelConfig", "KLControlConfig", "McoreActorConfig", "McoreEngineConfig", "MultiTurnConfig", "OptimizerConfig", "PolicyLossConfig",
           "RolloutConfig", "RolloutCorrectionConfig", "SamplingConfig", "from_config"]
