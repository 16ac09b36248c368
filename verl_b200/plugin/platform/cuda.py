"""NVIDIA platform (the product target: B200, compute capability 10.0). Reference: ``verl/plugin/platform/platform_cuda.py``."""

from __future__ import annotations

import os
from contextlib import contextmanager

import torch

from .base import PlatformBase
from .manager import PlatformRegistry

__all__ = ["PlatformCUDA"]


@PlatformRegistry.register("cuda")
class PlatformCUDA(PlatformBase):
    device_name = "cuda"
    vendor_name = "nvidia"

    @property
    def device_module(self):
        return torch.cuda

    def is_available(self) -> bool:
        return torch.cuda.is_available()

    def is_platform_available(self, use_smi_check: bool = False) -> bool:
        if self.is_available():
            return True
        return bool(use_smi_check) and self.check_smi_command("nvidia-smi")

    def set_allocator_settings(self, settings: str) -> None:
        if self.is_available():
            torch.cuda.memory._set_allocator_settings(settings)

    def get_device_capability(self, device_index: int = 0) -> tuple:
        return torch.cuda.get_device_capability(device_index) if self.is_available() else (None, None)

    def is_blackwell(self, device_index: int = 0) -> bool:
        """The hand-written kernels are sm_100a binaries; anything else cannot load them."""
        return self.get_device_capability(device_index)[0] == 10

    def get_device_uuid(self, device_id: int) -> str:
        return str(torch.cuda.get_device_properties(device_id).uuid) if self.is_available() else super().get_device_uuid(device_id)

    def communication_backend_name(self) -> str:
        return "nccl"

    def process_group_backend(self) -> str:
        return "cpu:gloo,cuda:nccl"

    def visible_devices_envvar(self) -> str:
        return "CUDA_VISIBLE_DEVICES"

    def is_ipc_supported(self) -> bool:
        return True                      # CUDA IPC handles carry the symmetric buffers between the ranks of one node

    def rollout_env_vars(self) -> dict:
        # the rollout engines decide device placement themselves; nothing may rewrite the visible-device list under them
        return {"NCCL_CUMEM_ENABLE": os.environ.get("NCCL_CUMEM_ENABLE", "0")}

    def ray_resource_name(self) -> str:
        return "GPU"

    def ray_noset_envvars(self) -> list:
        return ["RAY_EXPERIMENTAL_NOSET_CUDA_VISIBLE_DEVICES"]

    @contextmanager
    def nvtx_range(self, msg: str):
        if not self.is_available():
            yield
            return
        torch.cuda.nvtx.range_push(msg)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()

    def profiler_start(self) -> None:
        if self.is_available():
            torch.cuda.profiler.start()

    def profiler_stop(self) -> None:
        if self.is_available():
            torch.cuda.profiler.stop()

    def profiler_markers(self):
        n = torch.cuda.nvtx
        return (n.mark, n.range_push, n.range_pop, n.range) if self.is_available() else None

    def cudart(self):
        return torch.cuda.cudart() if self.is_available() else None
