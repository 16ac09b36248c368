"""Environment report for bug reports: Python / torch / CUDA / NCCL versions, GPUs with clocks and memory, NVLink peer
access matrix, the native extension's state (reference: ``scripts/diagnose.py``). Reads settings only."""

from __future__ import annotations

import platform
import shutil
import subprocess
import sys


def main():
    import torch

    print(f"python      {sys.version.split()[0]} on {platform.platform()}")
    print(f"torch       {torch.__version__} (cuda {torch.version.cuda}, nccl {'.'.join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else 'n/a'})")
    print(f"nvcc        {shutil.which('nvcc') or 'not found'}")
    from verl_b200.ops import _ext

    print(f"native ext  {'loaded' if _ext.available() else 'not available (CPU reference path)'}")
    if not torch.cuda.is_available():
        print("no CUDA device visible")
        return
    n = torch.cuda.device_count()
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        print(f"gpu {i}: {p.name} sm_{p.major}{p.minor} {p.total_memory / 2**30:.0f} GiB, {p.multi_processor_count} SMs")
    if n > 1:
        print("peer access:")
        for i in range(n):
            print("  " + " ".join("Y" if i == j or torch.cuda.can_device_access_peer(i, j) else "n" for j in range(n)))
    smi = shutil.which("nvidia-smi")
    if smi:
        q = "index,clocks.sm,clocks.max.sm,power.draw,power.limit,memory.used,clocks_event_reasons.active"
        print(subprocess.run([smi, f"--query-gpu={q}", "--format=csv"], capture_output=True, text=True).stdout)


if __name__ == "__main__":
    main()
