"""Process-level helpers of distributed workers: NUMA/CPU affinity next to the worker's GPU, process-group bootstrap.

``set_numa_affinity`` pins the calling process to the CPU cores that NVML reports as local to its GPU, so that pinned host
buffers, the dataloader threads and the launch thread stay on the socket the GPU hangs off. Only *queries* go to NVML
(``nvmlDeviceGetCpuAffinity``); the pinning itself is ``os.sched_setaffinity`` on this process — no device setting changes.

Reference: ``verl/utils/distributed.py:30-57`` (``set_numa_affinity`` through libnuma + pynvml), called from the worker
constructor (``verl/workers/engine_workers.py:92``).
"""

from __future__ import annotations

import os
from typing import Optional

__all__ = ["set_numa_affinity", "cpus_near_device", "initialize_global_process_group"]


def _visible_to_physical(local_index: int) -> int | str:
    """Index (or UUID) of the ``local_index``-th visible device in NVML's numbering."""
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if not vis:
        return local_index
    items = [v.strip() for v in vis.split(",") if v.strip()]
    if local_index >= len(items):
        return local_index
    it = items[local_index]
    return int(it) if it.lstrip("-").isdigit() else it


def cpus_near_device(local_index: int, nvml=None) -> list[int]:
    """CPU ids local to the GPU, from NVML's affinity bitmask (64 CPUs per word)."""
    if nvml is None:
        import pynvml as nvml
    nvml.nvmlInit()
    try:
        dev = _visible_to_physical(local_index)
        handle = nvml.nvmlDeviceGetHandleByUUID(dev) if isinstance(dev, str) else nvml.nvmlDeviceGetHandleByIndex(dev)
        words = (os.cpu_count() or 64) // 64 + 1
        mask = nvml.nvmlDeviceGetCpuAffinity(handle, words)
        return [w * 64 + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1]
    finally:
        nvml.nvmlShutdown()


def set_numa_affinity(local_index: Optional[int] = None, nvml=None, setter=None) -> Optional[list[int]]:
    """Pin this process to the CPUs near its GPU. Returns the CPU list, or None when nothing was changed (no GPU, NVML missing,
    an empty mask, or ``VERL_B200_NUMA_AFFINITY=0``). ``nvml`` / ``setter`` are injection points for tests."""
    if os.environ.get("VERL_B200_NUMA_AFFINITY", "1") == "0":
        return None
    if local_index is None:
        local_index = int(os.environ.get("LOCAL_RANK", "0"))
    try:
        cpus = cpus_near_device(local_index, nvml)
    except Exception as e:              # no driver, no NVML binding, index out of range: run unpinned
        print(f"[numa] affinity not set: {type(e).__name__}: {e}", flush=True)
        return None
    allowed = set(os.sched_getaffinity(0)) if setter is None and hasattr(os, "sched_getaffinity") else None
    if allowed is not None:
        cpus = [c for c in cpus if c in allowed]      # a container's cpuset may be narrower than the socket
    if not cpus:
        return None
    (setter or (lambda c: os.sched_setaffinity(0, c)))(cpus)
    return cpus


def initialize_global_process_group(timeout_s: int = 1800, numa: bool = True):
    """``torch.distributed`` bootstrap of one worker process from the torchrun environment: device selection, optional CPU
    pinning, global group on the platform's backend. Returns ``(local_rank, rank, world_size)``."""
    import datetime

    import torch.distributed as dist

    from verl_b200.plugin.platform import get_platform

    plat = get_platform()
    local_rank, rank, world = int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if plat.device_name != "cpu":
        plat.set_device(local_rank)
        if numa:
            set_numa_affinity(local_rank)
    if not dist.is_initialized():
        dist.init_process_group(plat.process_group_backend(), rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    return local_rank, rank, world
