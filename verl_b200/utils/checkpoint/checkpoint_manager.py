"""Checkpoint bookkeeping shared by all engines: what to save/load, retention, RNG state, tracker file, and the
"save before a known shutdown" (ESI) rule.

Parity target: ``verl/utils/checkpoint/checkpoint_manager.py`` (BaseCheckpointManager :29, RNG helpers :166-221,
find_latest_ckpt_path :222, get_checkpoint_tracker_filename :255, should_save_ckpt_esi :262).
"""

from __future__ import annotations

import os
import random
import shutil
import time
from typing import Optional

import numpy as np
import torch

__all__ = ["BaseCheckpointManager", "find_latest_ckpt_path", "get_checkpoint_tracker_filename", "should_save_ckpt_esi"]

TRACKER = "latest_checkpointed_iteration.txt"
ASYNC_PENDING = ".async_save_pending"        # present in a checkpoint directory while background writers may still be writing


class BaseCheckpointManager:
    """``save_contents`` / ``load_contents`` ⊆ {model, optimizer, extra, hf_model}."""

    def __init__(self, checkpoint_config=None):
        cfg = checkpoint_config or {}
        g = (lambda k, d: cfg.get(k, d)) if hasattr(cfg, "get") else (lambda k, d: getattr(cfg, k, d))
        self.save_contents = list(g("save_contents", ["model", "optimizer", "extra"]) or [])
        self.load_contents = list(g("load_contents", self.save_contents) or [])
        self.async_save = bool(g("async_save", False))
        self.previous_saved_paths: list[str] = []
        self.previous_global_step: Optional[int] = None

    @property
    def should_save_model(self):
        return "model" in self.save_contents

    @property
    def should_save_optimizer(self):
        return "optimizer" in self.save_contents

    @property
    def should_save_extra(self):
        return "extra" in self.save_contents

    @property
    def should_save_hf_model(self):
        return "hf_model" in self.save_contents

    @property
    def should_load_model(self):
        return "model" in self.load_contents

    @property
    def should_load_optimizer(self):
        return "optimizer" in self.load_contents

    @property
    def should_load_extra(self):
        return "extra" in self.load_contents

    def remove_previous_save_local_path(self, paths):
        for p in [paths] if isinstance(paths, str) else paths:
            if os.path.exists(p):
                shutil.rmtree(p, ignore_errors=True)

    def ensure_checkpoint_capacity(self, max_ckpt_to_keep: Optional[int]):
        """Delete oldest checkpoints so that, after the next save, at most ``max_ckpt_to_keep`` remain."""
        if isinstance(max_ckpt_to_keep, int) and max_ckpt_to_keep > 0 and len(self.previous_saved_paths) >= max_ckpt_to_keep:
            keep_start = len(self.previous_saved_paths) - max_ckpt_to_keep + 1
            self.remove_previous_save_local_path(self.previous_saved_paths[:keep_start])
            self.previous_saved_paths = self.previous_saved_paths[keep_start:]

    def register_checkpoint(self, path: str, max_ckpt_to_keep: Optional[int] = None):
        self.previous_saved_paths.append(path)

    # ---- asynchronous saves: a writer thread per rank; a checkpoint counts only once every rank has dropped its marker
    def wait_async_save(self):
        """Block until this rank's background writer (if any) has finished."""
        th = getattr(self, "_async_thread", None)
        if th is not None:
            th.join()
            self._async_thread = None

    @staticmethod
    def async_marker(path: str, rank: int) -> str:
        return os.path.join(path, f".async_done_rank_{rank}")

    @staticmethod
    def async_save_complete(path: str, world: int) -> bool:
        """True when ``path`` was not written asynchronously or all ``world`` writers have finished."""
        if not os.path.exists(os.path.join(path, ASYNC_PENDING)):
            return True
        return all(os.path.exists(BaseCheckpointManager.async_marker(path, r)) for r in range(world))

    @staticmethod
    def finish_async_save(path: str, world: int):
        """Rank 0, after ``async_save_complete``: remove the pending flag and the per-rank markers."""
        for r in range(world):
            try:
                os.remove(BaseCheckpointManager.async_marker(path, r))
            except OSError:
                pass
        try:
            os.remove(os.path.join(path, ASYNC_PENDING))
        except OSError:
            pass

    @staticmethod
    def local_mkdir_safe(path: str) -> str:
        os.makedirs(path, exist_ok=True)
        return path

    @staticmethod
    def get_rng_state() -> dict:
        st = {"cpu": torch.get_rng_state(), "numpy": np.random.get_state(), "random": random.getstate()}
        if torch.cuda.is_available():
            st["cuda"] = torch.cuda.get_rng_state()
        return st

    @staticmethod
    def load_rng_state(st: dict):
        torch.set_rng_state(st["cpu"])
        np.random.set_state(st["numpy"])
        random.setstate(st["random"])
        if torch.cuda.is_available() and "cuda" in st:
            torch.cuda.set_rng_state(st["cuda"])


def get_checkpoint_tracker_filename(root: str) -> str:
    return os.path.join(root, TRACKER)


def find_latest_ckpt_path(path: Optional[str], directory_format: str = "global_step_{}") -> Optional[str]:
    """Resolve ``<path>/global_step_N`` from the tracker file; None when nothing (valid) has been saved."""
    if path is None:
        return None
    tracker = get_checkpoint_tracker_filename(path)
    if not os.path.exists(tracker):
        return None
    try:
        it = int(open(tracker, "rb").read().decode().strip())
    except (ValueError, OSError):
        print(f"checkpoint tracker {tracker} is unreadable; ignoring it")
        return None
    ckpt = os.path.join(path, directory_format.format(it))
    if not os.path.exists(ckpt):
        print(f"checkpoint {ckpt} named by the tracker does not exist")
        return None
    return ckpt


def should_save_ckpt_esi(max_steps_duration: float, save_ckpt_duration: float = 60, redundant_time: float = 0) -> bool:
    """True when a platform-announced expiry (``MLP_CURRENT_CAPACITY_BLOCK_EXPIRATION_TIMESTAMP`` or
    ``SAGEMAKER_CURRENT_CAPACITY_BLOCK_EXPIRATION_TIMESTAMP``) is closer than one more step + one save + slack."""
    exp = os.getenv("MLP_CURRENT_CAPACITY_BLOCK_EXPIRATION_TIMESTAMP") or os.getenv("SAGEMAKER_CURRENT_CAPACITY_BLOCK_EXPIRATION_TIMESTAMP")
    if not exp:
        return False
    try:
        remaining = float(exp) - time.time()
    except ValueError:
        return False
    return remaining > 0 and max_steps_duration > 0 and remaining <= max_steps_duration + save_ckpt_duration + redundant_time
