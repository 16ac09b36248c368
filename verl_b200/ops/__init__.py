"""Hot-path operators: sm_100a kernels with PyTorch reference implementations as oracle."""

from . import _ext
from .functional import *  # noqa: F401,F403
