"""Worker base class: one process, one GPU, several colocated roles.

Reads its place in the group from the environment the launcher sets (``RANK``, ``WORLD_SIZE``, ``LOCAL_RANK``,
``MASTER_ADDR``, ``MASTER_PORT``) and keeps, per mesh name, the data-parallel coordinate used by n-d dispatch.
Parity target: ``verl/single_controller/base/worker.py:76-348``.
"""

from __future__ import annotations

import os
import socket
from dataclasses import dataclass

from .decorator import Dispatch, Execute, register

__all__ = ["Worker", "DistRankInfo", "DistGlobalInfo"]


@dataclass
class DistRankInfo:
    tp_rank: int = 0
    dp_rank: int = 0
    pp_rank: int = 0
    cp_rank: int = 0


@dataclass
class DistGlobalInfo:
    tp_size: int = 1
    dp_size: int = 1
    pp_size: int = 1
    cp_size: int = 1


class WorkerHelper:
    @staticmethod
    def _get_node_ip() -> str:
        return os.environ.get("VERL_NODE_IP", "127.0.0.1")

    @staticmethod
    def _get_free_port() -> int:
        with socket.socket() as s:
            s.bind(("", 0))
            return s.getsockname()[1]

    def get_availale_master_addr_port(self):
        return self._get_node_ip(), str(self._get_free_port())

    get_available_master_addr_port = get_availale_master_addr_port


class Worker(WorkerHelper):
    fused_worker_attr_name = "fused_worker_dict"

    def __init__(self, cuda_visible_devices=None) -> None:
        self._rank = int(os.environ.get("RANK", 0))
        self._world_size = int(os.environ.get("WORLD_SIZE", 1))
        self._local_rank = int(os.environ.get("LOCAL_RANK", self._rank))
        self._master_addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        self._master_port = os.environ.get("MASTER_PORT", "29500")
        self.fused_worker_dict = {}
        self.__dispatch_dp_rank: dict[str, int] = {}
        self.__collect_dp_rank: dict[str, bool] = {}
        self._setup_device()

    def _setup_device(self):
        try:
            import torch

            if torch.cuda.is_available():
                dev = self._local_rank % torch.cuda.device_count()
                torch.cuda.set_device(dev)
                from verl_b200.utils.distributed import set_numa_affinity

                self._cpu_affinity = set_numa_affinity(dev)       # stay on the socket the GPU hangs off (queries NVML only)
        except Exception:
            pass

    # ------------------------------------------------------------------ mesh registration for n-d dispatch
    def _register_dispatch_collect_info(self, mesh_name: str, dp_rank: int, is_collect: bool):
        if mesh_name in self.__dispatch_dp_rank:
            raise ValueError(f"mesh_name {mesh_name} has been registered")
        self.__dispatch_dp_rank[mesh_name] = dp_rank
        self.__collect_dp_rank[mesh_name] = is_collect

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def _query_dispatch_info(self, mesh_name: str):
        assert mesh_name in self.__dispatch_dp_rank, f"{mesh_name} is not registered in {type(self).__name__}"
        return self.__dispatch_dp_rank[mesh_name]

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def _query_collect_info(self, mesh_name: str):
        assert mesh_name in self.__collect_dp_rank, f"{mesh_name} is not registered in {type(self).__name__}"
        return self.__collect_dp_rank[mesh_name]

    # ------------------------------------------------------------------ properties
    @property
    def rank(self) -> int:
        return self._rank

    @property
    def world_size(self) -> int:
        return self._world_size

    @property
    def local_rank(self) -> int:
        return self._local_rank

    def get_master_addr_port(self):
        return self._master_addr, self._master_port

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def get_cuda_visible_devices(self):
        return os.environ.get("CUDA_VISIBLE_DEVICES", "")

    @register(dispatch_mode=Dispatch.DP_COMPUTE_PROTO_WITH_FUNC)
    def execute_with_func_generator(self, func, *args, **kwargs):
        return func(self, *args, **kwargs)

    @register(dispatch_mode=Dispatch.ALL_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def execute_func_rank_zero(self, func, *args, **kwargs):
        return func(*args, **kwargs)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def ping(self):
        return self._rank
