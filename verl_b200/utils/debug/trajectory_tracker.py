"""Dump intermediate tensors of a run to a directory (local or ``hdfs://``) without stalling the step that produced them.

``dump_data(obj, name)`` is a no-op unless ``VERL_ENABLE_TRACKER=1``.  When on, the object is serialised on the caller's thread (so later
in-place updates do not leak into the dump) and a background writer of this process stores it as ``<VERL_TRACKER_HDFS_DIR>/<name>.pt``;
``get_trajectory_tracker().wait()`` drains the writer and re-raises the first failure.  ``VERL_TRACKER_VERBOSE=1`` prints each file.

Reference: ``verl/utils/debug/trajectory_tracker.py:34-91`` (a detached Ray actor with the same three environment variables); here the
writer is a per-process thread, so a dump never crosses a process boundary before it reaches storage.
"""
from __future__ import annotations

import io
import os
import tempfile
import threading
from collections import deque
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Optional

import torch

from verl_b200.utils import fs


class TrajectoryTracker:
    def __init__(self, out_dir: str, verbose: bool = False, workers: int = 2):
        self.out_dir, self.verbose = out_dir, verbose
        if not fs.is_non_local(out_dir):
            self.out_dir = os.path.abspath(os.path.expanduser(out_dir))
        fs.makedirs(self.out_dir, exist_ok=True)
        self._pool = ThreadPoolExecutor(max_workers=workers, thread_name_prefix="trajectory-dump")
        self._pending: deque[Future] = deque()

    def _store(self, payload: bytes, name: str) -> str:
        dst = os.path.join(self.out_dir, f"{name}.pt")
        if fs.is_non_local(self.out_dir):
            with tempfile.NamedTemporaryFile(suffix=".pt", delete=False) as f:
                f.write(payload)
                tmp = f.name
            try:
                fs.copy(tmp, dst)
            finally:
                os.unlink(tmp)
        else:
            tmp = dst + ".part"
            with open(tmp, "wb") as f:
                f.write(payload)
            os.replace(tmp, dst)
        if self.verbose:
            print(f"trajectory tracker: wrote {dst} ({len(payload)} bytes)", flush=True)
        return dst

    def dump(self, data, name: str) -> Future:
        buf = io.BytesIO()
        torch.save(data, buf)
        fut = self._pool.submit(self._store, buf.getvalue(), name)
        self._pending.append(fut)
        return fut

    def wait(self) -> list[str]:
        out = []
        while self._pending:
            out.append(self._pending.popleft().result())
        return out

    wait_for_hdfs = wait


_tracker: Optional[TrajectoryTracker] = None
_lock = threading.Lock()


def get_trajectory_tracker() -> TrajectoryTracker:
    global _tracker
    out_dir = os.getenv("VERL_TRACKER_HDFS_DIR")
    if out_dir is None:
        raise RuntimeError("VERL_TRACKER_HDFS_DIR is not set")
    with _lock:
        if _tracker is None or _tracker.out_dir not in (out_dir, os.path.abspath(os.path.expanduser(out_dir))):
            _tracker = TrajectoryTracker(out_dir, verbose=os.getenv("VERL_TRACKER_VERBOSE", "0") == "1")
        return _tracker


def dump_data(data, name: str) -> Optional[Future]:
    if os.getenv("VERL_ENABLE_TRACKER", "0") != "1":
        return None
    return get_trajectory_tracker().dump(data, name)
