"""Device platform registry: one object answers every device-dependent question of the framework."""

from .base import PlatformBase  # noqa: F401
from .manager import PlatformRegistry, get_platform, set_platform  # noqa: F401
from .cuda import PlatformCUDA  # noqa: F401
from .cpu import PlatformCPU  # noqa: F401
