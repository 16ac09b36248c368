"""Loader for the in-tree sm_100a kernel library (``verl_b200/_C.so``).

On a machine with a CUDA device the library is mandatory: a missing or unloadable ``_C.so`` raises instead of
silently running a PyTorch fallback. On a CPU-only machine :func:`available` is False and callers use the plain
PyTorch reference implementations (which are also the numerical oracles of the GPU tests).
"""

from __future__ import annotations

import os
from pathlib import Path

import torch

_LIB = Path(__file__).resolve().parent.parent / "_C.so"
_loaded = False


def lib_path() -> Path:
    return _LIB


def available() -> bool:
    """True when the native kernels can be used (CUDA device present and library loaded)."""
    if os.environ.get("VERL_B200_DISABLE_NATIVE", "0") == "1":
        return False
    if not torch.cuda.is_available():
        return False
    load()
    return True


def load() -> None:
    global _loaded
    if _loaded:
        return
    if not _LIB.exists():
        raise RuntimeError(
            f"verl_b200 native library not found at {_LIB}; build it with `python -m verl_b200.csrc.build` "
            "(a CUDA device is present, refusing to fall back to PyTorch ops)"
        )
    torch.ops.load_library(str(_LIB))
    _loaded = True


def ops():
    load()
    return torch.ops.verl_b200


def check_status(where: str = "") -> None:
    """Raise if any kernel with bounded device-side waits gave up since the last check (synchronises)."""
    if not _loaded:
        return
    code = int(torch.ops.verl_b200.take_status())
    if code != 0:
        raise RuntimeError(f"verl_b200 kernel reported status {code & 0xFF} (block {code >> 8}) {where}")


_graph_launches = 0


def add_graph_launches(n: int) -> None:
    """Kernels replayed from a captured CUDA graph never pass through the bindings; account for them here."""
    global _graph_launches
    _graph_launches += int(n)


def launch_count() -> int:
    """Kernel-launching calls into the native library so far (direct calls + graph replays)."""
    if not _loaded:
        return 0
    return int(torch.ops.verl_b200.launch_count()) + _graph_launches
