"""Device helpers. This framework targets NVIDIA B200 only; CPU exists for tests and the gloo plumbing configuration.

Every answer comes from the registered platform object (``verl_b200.plugin.platform``), so an out-of-tree platform changes
them all at once. Parity target: ``verl/utils/device.py`` (get_device_name :96, get_torch_device :113, get_nccl_backend :135,
auto_set_device :151, get_device_capability :174, manual_seed :378).
"""

from __future__ import annotations

import os

import torch

from verl_b200.plugin.platform import get_platform

__all__ = ["is_cuda_available", "get_device_name", "get_device_id", "get_torch_device", "get_nccl_backend",
           "get_visible_devices_keyword", "set_expandable_segments", "get_default_backend", "get_resource_name", "get_vendor",
           "get_device_capability", "is_support_ipc", "is_device_available", "manual_seed", "manual_seed_all", "auto_set_device"]

is_cuda_available = torch.cuda.is_available()


def get_device_name() -> str:
    return get_platform().device_name


def get_vendor() -> str:
    return get_platform().vendor_name


def get_resource_name() -> str:
    return get_platform().ray_resource_name()


def get_device_id() -> int:
    return get_platform().current_device()


def get_torch_device():
    return get_platform().device_module


def get_nccl_backend() -> str:
    return get_platform().communication_backend_name()


def get_default_backend() -> str:
    """Backend string for the global process group: gloo for host objects, NCCL for device tensors."""
    return get_platform().process_group_backend()


def get_visible_devices_keyword() -> str:
    return get_platform().visible_devices_envvar()


def set_expandable_segments(enable: bool) -> None:
    get_platform().set_allocator_settings(f"expandable_segments:{enable}")


def get_device_capability(device_id: int = 0) -> tuple:
    return get_platform().get_device_capability(device_id)


def is_support_ipc() -> bool:
    return get_platform().is_ipc_supported()


def is_device_available() -> bool:
    return get_platform().device_name != "cpu" and get_platform().is_available()


def manual_seed(seed: int) -> None:
    get_platform().manual_seed(seed)


def manual_seed_all(seed: int) -> None:
    get_platform().manual_seed_all(seed)


def auto_set_device(config) -> None:
    """Write the detected device name into ``config.trainer.device`` when the config names another one."""
    want = get_device_name()
    tr = config.get("trainer") if hasattr(config, "get") else getattr(config, "trainer", None)
    if tr is None:
        return
    cur = tr.get("device", None) if hasattr(tr, "get") else getattr(tr, "device", None)
    if cur != want:
        if cur not in (None, "cpu", "cuda"):
            print(f"[device] trainer.device={cur!r} is not available here; using {want!r}", flush=True)
        try:
            tr["device"] = want
        except TypeError:
            setattr(tr, "device", want)


def local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
