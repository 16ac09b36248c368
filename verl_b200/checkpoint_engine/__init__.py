from .base import CheckpointEngine, CheckpointEngineRegistry, NaiveCheckpointEngine
from .delta_sharded import DeltaShardedEngine, delta_apply, delta_compact, tensor_checksum
from .nccl_engine import BucketedBroadcastEngine

__all__ = ["CheckpointEngine", "CheckpointEngineRegistry", "NaiveCheckpointEngine", "BucketedBroadcastEngine", "DeltaShardedEngine",
           "delta_apply", "delta_compact", "tensor_checksum"]
