"""Weight synchronisation between a trainer and rollout replicas that do not share memory with it.

A ``CheckpointEngine`` moves a stream of ``(name, tensor)`` pairs from the sending side (trainer rank 0 of the sync
group) to every receiver. Backends (``rollout.checkpoint_engine.backend``):

* ``naive``          same process: the pairs are handed over as they are (colocated replicas);
* ``nccl``           dense: tensors are packed into fixed-size uint8 buckets and broadcast over a torch.distributed group
                     (NCCL on GPUs → NVLink/NVSwitch, gloo on CPU), two buckets in flight, metadata as one small object
                     broadcast per bucket;
* ``delta_sharded``  sparse: only the elements whose bits changed since the previous sync travel, as
                     ``(int32 position, value)`` pairs with a checksum, falling back to dense when the delta is large.

Reference: ``verl/checkpoint_engine/base.py`` (registry, ``send_weights/receive_weights``), ``nccl_checkpoint_engine.py``
and ``delta_sync/*``.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Iterable, Iterator

import torch

__all__ = ["CheckpointEngine", "CheckpointEngineRegistry", "NaiveCheckpointEngine"]


class CheckpointEngineRegistry:
    _engines: dict[str, type] = {}

    @classmethod
    def register(cls, name: str):
        def deco(sub):
            cls._engines[name] = sub
            return sub

        return deco

    @classmethod
    def get(cls, name: str) -> type:
        if name not in cls._engines:
            from . import delta_sharded, nccl_engine  # noqa: F401 - populate

        if name not in cls._engines:
            raise ValueError(f"unknown checkpoint engine backend {name!r}; known: {sorted(cls._engines)}")
        return cls._engines[name]

    @classmethod
    def new(cls, name: str, **kwargs) -> "CheckpointEngine":
        return cls.get(name)(**kwargs)


class CheckpointEngine(ABC):
    @abstractmethod
    def send_weights(self, named_tensors: Iterable[tuple[str, torch.Tensor]]) -> dict:
        """Called on the source rank with the full model; returns transfer statistics."""

    @abstractmethod
    def receive_weights(self) -> Iterator[tuple[str, torch.Tensor]]:
        """Called on every other rank; yields tensors that are only valid until the next item is requested."""

    def finalize(self):
        pass


@CheckpointEngineRegistry.register("naive")
class NaiveCheckpointEngine(CheckpointEngine):
    """Sender and receiver are the same process: ``send_weights`` stores the iterator, ``receive_weights`` drains it."""

    def __init__(self, **kwargs):
        self._pending = None

    def send_weights(self, named_tensors):
        self._pending = named_tensors
        return {"backend": "naive"}

    def receive_weights(self):
        src, self._pending = self._pending, None
        yield from (src or ())
