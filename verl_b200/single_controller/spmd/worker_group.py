"""SPMD worker group: the controller program itself runs once per GPU (``torchrun``), every rank owns the local worker
and the "remote call" is a local call followed by an object all-gather, so each rank's controller sees exactly what a
central driver would. No RPC hop, no serialisation of tensors that stay on the rank.

This is the launch mode of ``bench.py`` and of multi-GPU tests; the spawned-process backend
(``verl_b200.single_controller.process``) gives the classic one-driver/N-workers topology of the reference
(``verl/single_controller/ray/base.py:426``) with the same ``@register`` semantics.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from ..base.worker_group import ClassWithInitArgs, ResourcePool, WorkerGroup, default_func_generator

__all__ = ["SPMDWorkerGroup", "init_spmd_process_group"]

_GLOO_GROUP = None


def init_spmd_process_group(timeout_s: int = 600):
    """Initialise torch.distributed from the torchrun environment (NCCL for tensors, gloo for host objects)."""
    global _GLOO_GROUP
    import datetime

    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if torch.cuda.is_available():
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dist.init_process_group("cpu:gloo,cuda:nccl", timeout=datetime.timedelta(seconds=timeout_s),
                                    device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
        else:
            dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=timeout_s))
    if dist.is_initialized() and _GLOO_GROUP is None:
        _GLOO_GROUP = dist.new_group(backend="gloo")
    return _GLOO_GROUP


class _Done:
    def __init__(self, v):
        self.v = v

    def result(self):
        return self.v


class SPMDWorkerGroup(WorkerGroup):
    def __init__(self, resource_pool: Optional[ResourcePool] = None, cls_with_init_args: Optional[ClassWithInitArgs] = None,
                 worker=None, **kwargs):
        super().__init__(resource_pool, **kwargs)
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self._world = dist.get_world_size() if dist.is_initialized() else 1
        self.gloo = init_spmd_process_group() if dist.is_initialized() else None
        self.worker = worker if worker is not None else cls_with_init_args()
        self._workers = list(range(self._world))
        self._bind_worker_method(type(self.worker), default_func_generator)

    @property
    def world_size(self) -> int:
        return self._world

    def _is_worker_alive(self, worker) -> bool:
        return True

    def _wait(self, output):
        return output

    def execute_all(self, method_name: str, *args, **kwargs):
        largs = [a[self.rank] for a in args]
        lkw = {k: v[self.rank] for k, v in kwargs.items()}
        out = getattr(self.worker, method_name)(*largs, **lkw)
        if self._world == 1:
            return [out]
        gathered = [None] * self._world
        dist.all_gather_object(gathered, out, group=self.gloo)
        return gathered

    def execute_rank_zero(self, method_name: str, *args, **kwargs):
        out = getattr(self.worker, method_name)(*args, **kwargs) if self.rank == 0 else None
        if self._world > 1:
            box = [out]
            dist.broadcast_object_list(box, src=0, group=self.gloo)
            out = box[0]
        return [out]
