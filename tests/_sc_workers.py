"""Worker classes used by the single-controller tests (must be importable by spawned processes)."""

import os
import sys
import time

import torch

from verl_b200.protocol import DataProto
from verl_b200.single_controller.base import Dispatch, Execute, Worker, register
from verl_b200.single_controller.base.decorator import make_nd_compute_dataproto_dispatch_fn


class EchoWorker(Worker):
    def __init__(self, scale=1):
        super().__init__()
        self.scale = scale
        # 2-way "model parallel": ranks (0,1) form dp group 0, (2,3) dp group 1; only even ranks return outputs
        self._register_dispatch_collect_info("train", dp_rank=self.rank // 2, is_collect=self.rank % 2 == 0)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def env(self):
        return {k: os.environ.get(k) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT", "WG_PREFIX")}

    @register(dispatch_mode=Dispatch.DP_COMPUTE_PROTO)
    def double(self, data: DataProto) -> DataProto:
        return DataProto.from_dict(tensors={"y": data.batch["x"] * 2 * self.scale, "rank": torch.full((len(data),), self.rank)})

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"))
    def nd(self, data: DataProto) -> DataProto:
        return DataProto.from_dict(tensors={"x": data.batch["x"], "rank": torch.full((len(data),), self.rank)})

    @register(dispatch_mode=Dispatch.ALL_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def only_zero(self, v):
        return (self.rank, v)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, blocking=False)
    def slow(self, t):
        time.sleep(t)
        return self.rank

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def boom(self):
        raise RuntimeError("intentional failure in worker")

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def die(self):
        os._exit(1)


class Adder(Worker):
    def __init__(self, k):
        super().__init__()
        self.k = k

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def add(self, v):
        return v + self.k


class EnvWorker(Worker):
    """Reports the launcher environment its process received."""

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def env(self):
        return (os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"])
