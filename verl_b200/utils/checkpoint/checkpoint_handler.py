"""Step folders, tracker file, retention and data position of a single-model training run.

One object owns everything around ``engine.save_checkpoint`` / ``engine.load_checkpoint`` that is not model state: where step ``N`` goes
(``<root>/global_step_N``), which step a restart resumes from (``resume_mode`` = ``auto`` | ``disable`` | ``resume_path``), how many step
folders stay on disk, and where in the data the run was.  The tracker file is replaced atomically and only after every rank has finished
writing, so it never names a half-written folder.  The data position is two integers (epoch, batches consumed in it): with a seeded
epoch-shuffling sampler that is enough to continue with exactly the batches an uninterrupted run would have seen, and `SkipFirst` gets
there without loading the skipped samples.

Covers the role of the reference's ``verl/utils/checkpoint/checkpoint_handler.py:49-234`` (``CheckpointHandler``: ``save_checkpoint``,
``load_checkpoint``, ``_determine_resume_path``, dataloader state) for SPMD (torchrun) trainers and for a controller that drives a worker
group.
"""
from __future__ import annotations

import os
import re
import shutil
from enum import Enum
from typing import Iterator, Optional

import torch
import torch.distributed as dist
from torch.utils.data import Sampler

from verl_b200.utils.checkpoint.checkpoint_manager import find_latest_ckpt_path, get_checkpoint_tracker_filename

DATA_STATE_FILE = "data.pt"
_STEP_RE = re.compile(r"global_step_(\d+)")


def extract_step(path: str) -> Optional[int]:
    """Step number of a ``…/global_step_N[/…]`` path, None when the path names no step folder."""
    m = _STEP_RE.search(str(path))
    return int(m.group(1)) if m else None


class OrchestrationMode(Enum):
    SPMD = "spmd"              # every rank holds a handler; rank 0 owns the tracker and the retention
    CONTROLLER = "controller"  # one handler on the driver; `engine` is a worker group whose calls fan out


class SkipFirst(Sampler[int]):
    """Wraps a sampler; the next iteration drops the first ``n`` indices, later iterations are untouched."""

    def __init__(self, sampler, n: int = 0):
        self.sampler, self.n = sampler, int(n)

    def skip_next(self, n: int):
        self.n = int(n)

    def set_epoch(self, epoch: int):
        if hasattr(self.sampler, "set_epoch"):
            self.sampler.set_epoch(epoch)

    def __iter__(self) -> Iterator[int]:
        n, self.n = self.n, 0
        for i, idx in enumerate(self.sampler):
            if i >= n:
                yield idx

    def __len__(self) -> int:
        return max(0, len(self.sampler) - self.n)


class CheckpointHandler:
    def __init__(self, engine, *, default_local_dir: str, max_ckpt_to_keep: Optional[int] = None, default_hdfs_dir: Optional[str] = None,
                 resume_mode: str = "auto", resume_from_path: Optional[str] = None, mode: OrchestrationMode = OrchestrationMode.SPMD,
                 rank: Optional[int] = None):
        if resume_mode not in ("auto", "disable", "resume_path"):
            raise ValueError(f"resume_mode must be auto, disable or resume_path, not {resume_mode!r}")
        self.engine = engine
        self.root = os.path.abspath(os.path.expanduser(default_local_dir))
        self.max_ckpt_to_keep = int(max_ckpt_to_keep) if max_ckpt_to_keep else None
        self.default_hdfs_dir = default_hdfs_dir
        self.resume_mode, self.resume_from_path = resume_mode, resume_from_path
        self.mode = mode
        if rank is not None:
            self.rank = int(rank)
        elif mode is OrchestrationMode.SPMD and dist.is_available() and dist.is_initialized():
            self.rank = dist.get_rank()
        else:
            self.rank = 0

    # ------------------------------------------------------------------ paths
    def step_dir(self, step: int) -> str:
        return os.path.join(self.root, f"global_step_{int(step)}")

    def saved_steps(self) -> list[int]:
        if not os.path.isdir(self.root):
            return []
        return sorted(s for s in (extract_step(d) for d in os.listdir(self.root) if os.path.isdir(os.path.join(self.root, d))) if s is not None)

    def resume_path(self) -> Optional[str]:
        """The folder a restart loads from under the configured mode; None for a fresh start."""
        if self.resume_mode == "disable":
            return None
        if self.resume_mode == "resume_path":
            p = self.resume_from_path
            if not p or extract_step(p) is None:
                raise ValueError("resume_mode=resume_path needs resume_from_path to name a global_step_N folder")
            p = os.path.abspath(os.path.expanduser(p))
            if not os.path.isdir(p):
                raise FileNotFoundError(f"resume_from_path {p} does not exist")
            return p
        return find_latest_ckpt_path(self.root)

    def _barrier(self):
        if self.mode is OrchestrationMode.SPMD and dist.is_available() and dist.is_initialized():
            dist.barrier()

    # ------------------------------------------------------------------ save / load
    def save_checkpoint(self, step: int, data_state: Optional[dict] = None) -> str:
        path = self.step_dir(step)
        hdfs = os.path.join(self.default_hdfs_dir, f"global_step_{int(step)}") if self.default_hdfs_dir else None
        self.engine.save_checkpoint(path, hdfs_path=hdfs, global_step=int(step))
        if self.rank == 0 and data_state is not None:
            os.makedirs(path, exist_ok=True)
            torch.save(dict(data_state), os.path.join(path, DATA_STATE_FILE))
        self._barrier()   # every rank's files are on disk before the tracker moves
        if self.rank == 0:
            tracker = get_checkpoint_tracker_filename(self.root)
            tmp = tracker + ".tmp"
            with open(tmp, "w") as f:
                f.write(str(int(step)))
                f.flush()
                os.fsync(f.fileno())
            os.replace(tmp, tracker)
            if self.max_ckpt_to_keep:
                for old in self.saved_steps()[:-self.max_ckpt_to_keep]:
                    if old != int(step):
                        shutil.rmtree(self.step_dir(old), ignore_errors=True)
        self._barrier()
        return path

    def load_checkpoint(self) -> tuple[int, Optional[dict]]:
        """Loads the resume folder into the engine; returns (step, data state) — (0, None) for a fresh start."""
        path = self.resume_path()
        if path is None:
            return 0, None
        self.engine.load_checkpoint(path)
        f = os.path.join(path, DATA_STATE_FILE)
        data_state = torch.load(f, weights_only=False) if os.path.exists(f) else None
        return int(extract_step(path)), data_state
