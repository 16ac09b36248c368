"""Nsight Systems around worker processes.

``nsys`` profiles a process from the outside, so the worker launcher has to start the worker as ``nsys profile <options>
python ...``. :func:`nsys_command_prefix` turns the ``global_profiler.global_tool_config.nsys.*_nsight_options`` mapping of
the trainer config into that prefix (one report per process, capture bounded by ``cudaProfilerApi`` so that
``DistProfiler.start/stop`` decide what is recorded), :func:`wrap_worker_command` applies it to a worker command line, and
:func:`relocate_results` moves the finished ``*.nsys-rep`` files of this process into ``save_path`` under names that carry
the host and the role.

Reference: the Ray ``runtime_env["nsight"]`` wrapping in ``verl/trainer/main_ppo_v0.py`` / ``verl/single_controller/ray/base.py``
and ``NsightSystemsProfiler.relocate_results`` (``verl/utils/profiler/nvtx_profile.py:130-218``).
"""

from __future__ import annotations

import glob
import os
import shutil
import socket
from typing import Optional, Sequence

__all__ = ["DEFAULT_WORKER_OPTIONS", "nsys_available", "nsys_command_prefix", "wrap_worker_command", "relocate_results"]

DEFAULT_WORKER_OPTIONS = {"trace": "cuda,nvtx,cublas,ucx", "cuda-memory-usage": "true", "cuda-graph-trace": "graph",
                          "capture-range": "cudaProfilerApi", "capture-range-end": None, "kill": "none"}


def nsys_available() -> bool:
    return shutil.which("nsys") is not None


def nsys_command_prefix(options: Optional[dict], output: str, discrete: bool = False) -> list:
    """``["nsys", "profile", "--trace=...", ..., "-o", output]``. ``None`` values drop an option (its nsys default
    applies); with ``discrete`` every capture range becomes its own report (``capture-range-end=repeat``)."""
    opts = dict(DEFAULT_WORKER_OPTIONS)
    opts.update(options or {})
    if discrete and not opts.get("capture-range-end"):
        opts["capture-range-end"] = "repeat"
    cmd = ["nsys", "profile"]
    for k, v in opts.items():
        if v is None:
            continue
        cmd.append(f"--{k}={str(v).lower() if isinstance(v, bool) else v}")
    return cmd + ["--force-overwrite=true", "-o", output]


def wrap_worker_command(cmd: Sequence[str], options: Optional[dict], out_dir: str, role: str = "worker", rank: int = 0, discrete: bool = False) -> list:
    """The same worker command under ``nsys profile``; the report goes to ``out_dir/<role>_rank<rank>_<host>``."""
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, f"{role}_rank{rank}_{socket.gethostname()}")
    return nsys_command_prefix(options, out, discrete) + list(cmd)


def relocate_results(save_path: Optional[str], source_dir: str, *, pid: Optional[int] = None, role: Optional[str] = None) -> list:
    """Move this process's reports (``worker_process_<pid>.*`` under ``source_dir``: the final ``.nsys-rep`` and, while a
    session is still open, ``.qdstrm`` intermediates) into ``save_path`` as ``[<role>_]<host>_<name>``. Safe to call more
    than once; returns the destination paths that were moved."""
    if not save_path:
        return []
    pid = os.getpid() if pid is None else pid
    found = sorted(glob.glob(os.path.join(source_dir, f"worker_process_{pid}.*")))
    if not found:
        return []
    os.makedirs(save_path, exist_ok=True)
    host, prefix, moved = socket.gethostname(), (f"{role}_" if role else ""), []
    for src in found:
        dst = os.path.join(save_path, f"{prefix}{host}_{os.path.basename(src)}")
        try:
            shutil.move(src, dst)
            moved.append(dst)
        except (FileNotFoundError, OSError):
            continue
    return moved
