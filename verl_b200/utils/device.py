"""Device helpers. This framework targets NVIDIA B200 only; CPU exists for tests and the gloo plumbing configuration.

Parity target: ``verl/utils/device.py`` (get_device_name :96, get_torch_device :113, get_nccl_backend :135) and the
CUDA platform of ``verl/plugin/platform/platform_cuda.py``.
"""

from __future__ import annotations

import os

import torch

__all__ = ["is_cuda_available", "get_device_name", "get_device_id", "get_torch_device", "get_nccl_backend",
           "get_visible_devices_keyword", "set_expandable_segments", "get_default_backend"]

is_cuda_available = torch.cuda.is_available()


def get_device_name() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def get_device_id() -> int:
    return torch.cuda.current_device() if torch.cuda.is_available() else 0


def get_torch_device():
    return torch.cuda if torch.cuda.is_available() else torch.cpu


def get_nccl_backend() -> str:
    return "nccl" if torch.cuda.is_available() else "gloo"


def get_default_backend() -> str:
    """Backend string for the global process group: gloo for host objects, NCCL for device tensors."""
    return "cpu:gloo,cuda:nccl" if torch.cuda.is_available() else "gloo"


def get_visible_devices_keyword() -> str:
    return "CUDA_VISIBLE_DEVICES"


def set_expandable_segments(enable: bool) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._set_allocator_settings(f"expandable_segments:{enable}")


def local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
