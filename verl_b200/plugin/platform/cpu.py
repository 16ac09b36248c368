"""Host platform: what the test-suite and the gloo plumbing run on."""

from __future__ import annotations

import torch

from .base import PlatformBase
from .manager import PlatformRegistry

__all__ = ["PlatformCPU"]


@PlatformRegistry.register("cpu")
class PlatformCPU(PlatformBase):
    device_name = "cpu"
    vendor_name = "host"

    @property
    def device_module(self):
        return torch.cpu

    def is_available(self) -> bool:
        return True

    def current_device(self) -> int:
        return 0

    def device_count(self) -> int:
        return 1

    def set_device(self, device_index: int) -> None:
        return None

    def synchronize(self, device_index=None) -> None:
        return None

    def manual_seed(self, seed: int) -> None:
        torch.manual_seed(seed)

    def manual_seed_all(self, seed: int) -> None:
        torch.manual_seed(seed)

    def empty_cache(self) -> None:
        return None

    def set_allocator_settings(self, settings: str) -> None:
        return None

    def get_device_capability(self, device_index: int = 0) -> tuple:
        return (None, None)

    def communication_backend_name(self) -> str:
        return "gloo"

    def visible_devices_envvar(self) -> str:
        return "CUDA_VISIBLE_DEVICES"

    def is_ipc_supported(self) -> bool:
        return False

    def ray_resource_name(self) -> str:
        return "CPU"

    def ray_resource_options(self, num_gpus: float) -> dict:
        return {"num_cpus": max(1, int(num_gpus))}
