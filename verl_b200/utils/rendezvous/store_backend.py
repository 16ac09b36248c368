"""Building an extra communicator between processes that are NOT one torch.distributed world (e.g. trainer ranks plus
standalone rollout replicas for weight broadcast). The reference exchanges an NCCL unique id through a named Ray actor
and creates a cupy communicator (``verl/utils/rendezvous/ray_backend.py:35-101``); here a ``torch.distributed.TCPStore``
on 127.0.0.1 (or a given host) plays the id store and the communicator is a second, independent process group.
"""

from __future__ import annotations

import datetime
from typing import Optional

import torch.distributed as dist

__all__ = ["IdStore", "create_process_group_from_store"]


class IdStore:
    """Tiny key/value rendezvous: rank 0 hosts, everyone else connects."""

    def __init__(self, host: str, port: int, world_size: int, is_master: bool, timeout_s: int = 300):
        self.store = dist.TCPStore(host, port, world_size, is_master=is_master, timeout=datetime.timedelta(seconds=timeout_s),
                                   wait_for_workers=False)

    def set(self, key: str, value: bytes):
        self.store.set(key, value)

    def get(self, key: str) -> bytes:
        return self.store.get(key)


def create_process_group_from_store(host: str, port: int, rank: int, world_size: int, backend: Optional[str] = None, group_name: str = "weight_sync",
                                    timeout_s: int = 300):
    """A process group independent of the default one (which may not exist in this process at all). Uses the
    non-default-group constructor so that trainer ranks can be members of their training world AND of this group."""
    import torch

    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    store = dist.TCPStore(host, port, world_size, is_master=(rank == 0), timeout=datetime.timedelta(seconds=timeout_s), wait_for_workers=False)
    prefixed = dist.PrefixStore(group_name, store)
    from torch.distributed.distributed_c10d import _new_process_group_helper, _world  # noqa: F401

    if not dist.is_initialized():
        dist.init_process_group(backend, store=prefixed, rank=rank, world_size=world_size, timeout=datetime.timedelta(seconds=timeout_s))
        return dist.group.WORLD
    pg, _ = _new_process_group_helper(world_size, rank, [], backend, prefixed, group_name=group_name, timeout=datetime.timedelta(seconds=timeout_s))
    return pg
