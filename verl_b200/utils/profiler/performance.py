"""Timers and memory loggers. Device timing uses CUDA events on the launching stream and reduces with MAX over ranks.

Reference: ``verl/utils/profiler/performance.py`` (log_gpu_memory_usage :63, GPUMemoryLogger :85, simple_timer :155,
marked_timer :172, reduce_timing :198).
"""

from __future__ import annotations

import logging
import time
from contextlib import contextmanager
from typing import Optional

import torch
import torch.distributed as dist

__all__ = ["log_gpu_memory_usage", "GPUMemoryLogger", "simple_timer", "marked_timer", "reduce_timing", "DeviceTimer"]


def _mem_info(unit="GB", precision=2):
    div = {"GB": 1024**3, "MB": 1024**2, "KB": 1024}[unit]
    if not torch.cuda.is_available():
        return "0", "0", "0", "0"
    free, total = torch.cuda.mem_get_info()
    f = lambda v: f"{v / div:.{precision}f}"
    return f(torch.cuda.memory_allocated()), f(torch.cuda.memory_reserved()), f(total - free), f(total)


def log_gpu_memory_usage(head: str, logger: Optional[logging.Logger] = None, level=logging.DEBUG, rank: int = 0):
    if dist.is_initialized() and rank is not None and dist.get_rank() != rank:
        return
    a, r, u, t = _mem_info()
    msg = f"{head}, memory allocated (GB): {a}, memory reserved (GB): {r}, device memory used/total (GB): {u}/{t}"
    (logger.log(level, msg) if logger else print(msg))


class GPUMemoryLogger:
    """Decorator logging memory before and after the wrapped call."""

    def __init__(self, role: str, logger: Optional[logging.Logger] = None, level=logging.DEBUG, log_only_rank_0: bool = True):
        self.role, self.logger, self.level, self.rank0 = role, logger, level, log_only_rank_0

    def __call__(self, fn):
        from functools import wraps

        @wraps(fn)
        def inner(*a, **k):
            log_gpu_memory_usage(f"[{self.role}] Before {fn.__name__}", self.logger, self.level, 0 if self.rank0 else None)
            out = fn(*a, **k)
            log_gpu_memory_usage(f"[{self.role}] After {fn.__name__}", self.logger, self.level, 0 if self.rank0 else None)
            return out

        return inner


@contextmanager
def simple_timer(name: str, timing_raw: dict):
    t0 = time.perf_counter()
    yield
    timing_raw[name] = timing_raw.get(name, 0.0) + time.perf_counter() - t0


@contextmanager
def marked_timer(name: str, timing_raw: dict, color: Optional[str] = None, **kwargs):
    """Wall timer that also opens an NVTX range (visible in Nsight Systems)."""
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
    try:
        with simple_timer(name, timing_raw):
            yield
    finally:
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()


class DeviceTimer:
    """CUDA-event timer: ``with DeviceTimer() as t: ...; t.ms`` (device time on the current stream); ``max_over_ranks``
    gives the figure multi-GPU numbers must be quoted with."""

    def __enter__(self):
        self.s, self.e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        self.s.record()
        return self

    def __exit__(self, *exc):
        self.e.record()
        torch.cuda.synchronize()
        self.ms = self.s.elapsed_time(self.e)
        return False

    def max_over_ranks(self, group=None) -> float:
        t = torch.tensor([self.ms], device="cuda", dtype=torch.float64)
        if dist.is_initialized():
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return float(t.item())


def reduce_timing(timing_raw: dict, reduce_op=None) -> dict:
    """All-reduce (default: mean) every timing across ranks."""
    if not dist.is_initialized() or not timing_raw:
        return timing_raw
    keys = sorted(timing_raw)
    dev = "cuda" if torch.cuda.is_available() and dist.get_backend() != "gloo" else "cpu"
    t = torch.tensor([timing_raw[k] for k in keys], dtype=torch.float64, device=dev)
    op = reduce_op or dist.ReduceOp.SUM
    dist.all_reduce(t, op=op)
    if reduce_op is None:
        t /= dist.get_world_size()
    return {k: float(v) for k, v in zip(keys, t.tolist())}
