"""What the framework needs to know about the device it runs on, in one interface.

This build has exactly one accelerator target (NVIDIA B200, sm_100a) plus the CPU for tests; the interface exists so that
device questions (which torch module, which collective backend, which environment variable hides devices, whether peer
memory can be shared between processes, how to mark profiler ranges) are asked in one place and so that an out-of-tree
platform can register itself without touching core code.

Reference: ``verl/plugin/platform/platform_base.py:20-290`` (the abstract surface) — Ray resource naming included, since the
process-based controller of this framework uses the same strings in its resource pools.
"""

from __future__ import annotations

import abc
import shutil
import subprocess
from contextlib import contextmanager
from types import ModuleType
from typing import Any, Optional

__all__ = ["PlatformBase"]


class PlatformBase(abc.ABC):
    # ------------------------------------------------------------------ identity
    @property
    @abc.abstractmethod
    def device_name(self) -> str: ...

    @property
    @abc.abstractmethod
    def vendor_name(self) -> str: ...

    @property
    @abc.abstractmethod
    def device_module(self) -> ModuleType: ...

    @abc.abstractmethod
    def is_available(self) -> bool: ...

    @staticmethod
    def check_smi_command(cmd: str, timeout: float = 10.0) -> bool:
        """True when the vendor's management tool exists and answers a plain listing (read-only)."""
        exe = shutil.which(cmd)
        if exe is None:
            return False
        try:
            return subprocess.run([exe, "-L"], capture_output=True, timeout=timeout).returncode == 0
        except Exception:
            return False

    def is_platform_available(self, use_smi_check: bool = False) -> bool:
        return self.is_available()

    # ------------------------------------------------------------------ device handling
    def current_device(self) -> int:
        return self.device_module.current_device()

    def device_count(self) -> int:
        return self.device_module.device_count()

    def set_device(self, device_index: int) -> None:
        self.device_module.set_device(device_index)

    def synchronize(self, device_index: Optional[int] = None) -> None:
        self.device_module.synchronize(device_index) if device_index is not None else self.device_module.synchronize()

    def manual_seed(self, seed: int) -> None:
        self.device_module.manual_seed(seed)

    def manual_seed_all(self, seed: int) -> None:
        self.device_module.manual_seed_all(seed)

    def empty_cache(self) -> None:
        self.device_module.empty_cache()

    @abc.abstractmethod
    def set_allocator_settings(self, settings: str) -> None: ...

    @abc.abstractmethod
    def get_device_capability(self, device_index: int = 0) -> tuple: ...

    def get_device_uuid(self, device_id: int) -> str:
        return f"{self.device_name}-{device_id}"

    # ------------------------------------------------------------------ communication / process layout
    @abc.abstractmethod
    def communication_backend_name(self) -> str: ...

    def process_group_backend(self) -> str:
        """Backend string for the global group (host objects + device tensors)."""
        return self.communication_backend_name()

    @abc.abstractmethod
    def visible_devices_envvar(self) -> str: ...

    @abc.abstractmethod
    def is_ipc_supported(self) -> bool: ...

    def supports_colocated_worker_groups(self) -> bool:
        return True

    def rollout_env_vars(self) -> dict:
        return {}

    def get_collective_module(self) -> Any:
        import torch.distributed as dist

        return dist

    # ------------------------------------------------------------------ resource naming (pools of the single controller)
    @abc.abstractmethod
    def ray_resource_name(self) -> str: ...

    def ray_noset_envvars(self) -> list:
        return []

    def ray_resource_options(self, num_gpus: float) -> dict:
        return {"num_gpus": num_gpus} if self.ray_resource_name() == "GPU" else {"resources": {self.ray_resource_name(): num_gpus}}

    # ------------------------------------------------------------------ profiling hooks
    @contextmanager
    def nvtx_range(self, msg: str):
        yield

    def profiler_start(self) -> None:
        return None

    def profiler_stop(self) -> None:
        return None

    def profiler_markers(self):
        return None

    def apply_model_patches(self, model_type: str) -> None:
        return None

    def cudart(self) -> Any:
        return None
