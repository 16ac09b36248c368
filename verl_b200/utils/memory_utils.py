"""GPU memory housekeeping (reference: ``verl/utils/memory_utils.py:32-260``): aggressive cache release between phases,
memory snapshots for post-mortem analysis, a background sampler of allocator statistics."""

from __future__ import annotations

import gc
import os
import threading
import time
from typing import Optional

import torch

__all__ = ["aggressive_empty_cache", "reset_memory_stats", "get_memory_info", "log_memory_usage", "MemorySnapshotSampler", "enable_memory_history",
           "dump_memory_snapshot"]


def aggressive_empty_cache(force_sync: bool = True, max_retries: int = 3) -> float:
    """gc + empty_cache until the reserved size stops shrinking; returns the freed GB."""
    if not torch.cuda.is_available():
        gc.collect()
        return 0.0
    before = torch.cuda.memory_reserved()
    for _ in range(max_retries):
        gc.collect()
        torch.cuda.empty_cache()
        if force_sync:
            torch.cuda.synchronize()
        cur = torch.cuda.memory_reserved()
        if before - cur < (1 << 20):
            break
        before_loop = cur  # noqa: F841
    return (before - torch.cuda.memory_reserved()) / 1e9


def reset_memory_stats():
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()
        torch.cuda.reset_accumulated_memory_stats()


def get_memory_info() -> dict:
    if not torch.cuda.is_available():
        return {}
    free, total = torch.cuda.mem_get_info()
    return {"allocated_gb": torch.cuda.memory_allocated() / 1e9, "reserved_gb": torch.cuda.memory_reserved() / 1e9,
            "max_allocated_gb": torch.cuda.max_memory_allocated() / 1e9, "free_gb": free / 1e9, "total_gb": total / 1e9}


def log_memory_usage(head: str = "", rank: Optional[int] = 0, logger=None):
    import torch.distributed as dist

    if rank is not None and dist.is_initialized() and dist.get_rank() != rank:
        return
    info = get_memory_info()
    msg = f"{head} " + ", ".join(f"{k}={v:.2f}" for k, v in info.items())
    (logger.info if logger else print)(msg)


def enable_memory_history(max_entries: int = 100000):
    if torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(max_entries=max_entries)


def dump_memory_snapshot(out_dir: str, tag: str = "snapshot") -> Optional[str]:
    if not torch.cuda.is_available():
        return None
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, f"{tag}_rank{os.environ.get('RANK', '0')}.pickle")
    torch.cuda.memory._dump_snapshot(path)
    return path


class MemorySnapshotSampler:
    """Background thread sampling allocator statistics every ``interval_s`` (cheap; no device synchronisation)."""

    def __init__(self, interval_s: float = 1.0):
        self.interval_s, self.samples = interval_s, []
        self._stop = threading.Event()
        self._th: Optional[threading.Thread] = None

    def start(self):
        def run():
            while not self._stop.wait(self.interval_s):
                self.samples.append((time.time(), get_memory_info()))

        self._th = threading.Thread(target=run, daemon=True)
        self._th.start()
        return self

    def stop(self) -> list:
        self._stop.set()
        if self._th:
            self._th.join(timeout=5)
        return self.samples
