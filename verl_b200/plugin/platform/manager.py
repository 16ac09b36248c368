"""Registry and process-wide singleton of the device platform.

Selection order: ``VERL_B200_PLATFORM`` (a registered name) → CUDA when a device is visible → CPU. Out-of-tree platforms
register with ``@PlatformRegistry.register("name")`` before the first ``get_platform()`` call.

Reference: ``verl/plugin/platform/platform_manager.py:29-174``.
"""

from __future__ import annotations

import os
from typing import Optional

from .base import PlatformBase

__all__ = ["PlatformRegistry", "get_platform", "set_platform"]


class PlatformRegistry:
    _platforms: dict = {}

    @classmethod
    def register(cls, platform: str):
        def deco(platform_cls):
            if not (isinstance(platform_cls, type) and issubclass(platform_cls, PlatformBase)):
                raise TypeError(f"{platform_cls!r} must be a subclass of PlatformBase")
            cls._platforms[platform] = platform_cls
            return platform_cls

        return deco

    @classmethod
    def get(cls, name: str):
        return cls._platforms.get(name)

    @classmethod
    def registered_names(cls) -> tuple:
        return tuple(cls._platforms)


_current: Optional[PlatformBase] = None


def _detect_platform_name() -> str:
    forced = os.environ.get("VERL_B200_PLATFORM")
    if forced:
        if PlatformRegistry.get(forced) is None:
            raise ValueError(f"VERL_B200_PLATFORM={forced!r} is not registered (known: {PlatformRegistry.registered_names()})")
        return forced
    import torch

    return "cuda" if torch.cuda.is_available() else "cpu"


def get_platform() -> PlatformBase:
    global _current
    if _current is None:
        from . import cpu, cuda  # noqa: F401  (registers the built-in platforms)

        _current = PlatformRegistry.get(_detect_platform_name())()
    return _current


def set_platform(platform: Optional[PlatformBase]) -> None:
    """Install a platform object (tests, out-of-tree back ends); ``None`` re-runs the detection on the next ``get_platform()``."""
    global _current
    if platform is not None and not isinstance(platform, PlatformBase):
        raise TypeError("set_platform expects a PlatformBase instance")
    _current = platform
