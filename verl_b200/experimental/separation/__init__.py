"""Actor workers whose weights can be parked on, and brought back from, host memory under a key."""
from verl_b200.experimental.separation.engine_workers import DetachActorWorker

__all__ = ["DetachActorWorker"]
