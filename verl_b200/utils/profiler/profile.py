"""Per-worker profiler facade: rank/step filtering, tool selection (nsys ranges, torch.profiler, CUDA memory history),
``annotate`` decorator for worker methods and the ``start/stop`` RPCs the trainer calls around a step.

Reference: ``verl/utils/profiler/profile.py`` (DistProfiler :88-380, DistProfilerExtension :428-463), nvtx helpers
(``nvtx_profile.py:43-153``), torch profiler (``torch_profile.py:117-256``), memory (``torch_memory_profile.py:29``).
"""

from __future__ import annotations

import functools
import os
import subprocess
from typing import Callable, Optional

import torch

from verl_b200.single_controller.base import Dispatch, register

from .config import ProfilerConfig

__all__ = ["DistProfiler", "DistProfilerExtension", "mark_start_range", "mark_end_range", "mark_annotate"]


def mark_start_range(message: Optional[str] = None, **kwargs):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(message or "range")
    return message


def mark_end_range(range_id=None):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


def mark_annotate(message: Optional[str] = None, **kwargs) -> Callable:
    def deco(fn):
        @functools.wraps(fn)
        def inner(*a, **k):
            mark_start_range(message or fn.__name__)
            try:
                return fn(*a, **k)
            finally:
                mark_end_range()

        return inner

    return deco


class _TorchTool:
    def __init__(self, rank: int, cfg: ProfilerConfig):
        self.rank, self.cfg = rank, cfg
        self.prof = None

    def start(self, **kw):
        tc = self.cfg.tool_config or {}
        acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        self.prof = torch.profiler.profile(activities=acts, with_stack=bool(tc.get("with_stack", False)), record_shapes=bool(tc.get("record_shapes", False)))
        self.prof.start()

    def stop(self):
        if self.prof is None:
            return
        self.prof.stop()
        os.makedirs(self.cfg.save_path, exist_ok=True)
        self.prof.export_chrome_trace(os.path.join(self.cfg.save_path, f"trace_rank{self.rank}.json"))
        self.prof = None


class _NsysTool:
    """Capture ranges for an ``nsys profile --capture-range=cudaProfilerApi`` session wrapped around the process."""

    def __init__(self, rank, cfg):
        self.discrete = bool((cfg.tool_config or {}).get("discrete", False))

    def start(self, **kw):
        if torch.cuda.is_available() and not self.discrete:
            torch.cuda.profiler.start()

    def stop(self):
        if torch.cuda.is_available() and not self.discrete:
            torch.cuda.profiler.stop()


class _PrecisionTool:
    """Per-module numeric fingerprints of the stages named in ``tool_config.stages`` (see ``precision_debugger.py``); the
    worker passes ``stage=`` and ``model=`` to ``DistProfiler.start``."""

    def __init__(self, rank, cfg):
        from .precision_debugger import PrecisionDebugger

        tc = cfg.tool_config or {}
        self.dbg = PrecisionDebugger(rank, cfg.save_path, tc.get("stages"), bool(tc.get("strict", False)))
        self._model = None

    def start(self, stage: str = "actor_update", model=None, step: int = 0, **kw):
        if model is not None and self.dbg.start(stage, model, step):
            self._model = model

    def stop(self):
        self.dbg.stop(self._model)
        self._model = None


class _MemoryTool:
    def __init__(self, rank, cfg):
        self.rank, self.cfg = rank, cfg

    def start(self, **kw):
        if torch.cuda.is_available():
            tc = self.cfg.tool_config or {}
            torch.cuda.memory._record_memory_history(max_entries=int(tc.get("trace_alloc_max_entries", 100000)))

    def stop(self):
        if torch.cuda.is_available():
            os.makedirs(self.cfg.save_path, exist_ok=True)
            torch.cuda.memory._dump_snapshot(os.path.join(self.cfg.save_path, f"memory_rank{self.rank}.pickle"))
            torch.cuda.memory._record_memory_history(enabled=None)


class DistProfiler:
    def __init__(self, rank: int, config: Optional[ProfilerConfig] = None, tool_config=None, **kwargs):
        self.rank = rank
        self.config = config or ProfilerConfig()
        self.enabled = bool(self.config.enable and self.config.tool) and (self.config.all_ranks or rank in self.config.ranks)
        impl = {"torch": _TorchTool, "nsys": _NsysTool, "torch_memory": _MemoryTool, "precision_debugger": _PrecisionTool}.get(self.config.tool)
        self._impl = impl(rank, self.config) if (self.enabled and impl) else None
        self._running = False

    def check_enable(self) -> bool:
        return self.enabled

    def start(self, **kwargs):
        if self._impl is not None and not self._running:
            self._impl.start(**kwargs)
            self._running = True

    def stop(self):
        if self._impl is not None and self._running:
            self._impl.stop()
            self._running = False
            self._run_finish_hook()

    def relocate_results(self, source_dir: str, role: Optional[str] = None) -> list:
        """nsys writes its reports where the launcher pointed it; move this process's files under ``save_path``."""
        if self.config.tool != "nsys":
            return []
        from .nsys import relocate_results

        return relocate_results(self.config.save_path, source_dir, role=role)

    def _run_finish_hook(self):
        cmd = self.config.finish_hook_cmd
        if cmd and self.rank == 0:
            subprocess.run(cmd, shell=True, check=False, env=dict(os.environ, VERL_PROFILE_SAVE_PATH=self.config.save_path))

    @classmethod
    def annotate(cls, message: Optional[str] = None, color: Optional[str] = None, role: Optional[str] = None, **kwargs) -> Callable:
        """Decorator for worker methods: NVTX range, and in discrete mode a separate capture per call."""
        def deco(fn):
            @functools.wraps(fn)
            def inner(self_, *a, **k):
                prof = getattr(self_, "profiler", None)
                discrete = prof is not None and prof.enabled and prof.config.tool == "nsys" and (prof.config.tool_config or {}).get("discrete", False)
                if discrete and torch.cuda.is_available():
                    torch.cuda.profiler.start()
                mark_start_range(message or f"{role or type(self_).__name__}.{fn.__name__}")
                try:
                    return fn(self_, *a, **k)
                finally:
                    mark_end_range()
                    if discrete and torch.cuda.is_available():
                        torch.cuda.profiler.stop()

            return inner

        return deco


class DistProfilerExtension:
    """Mixin for workers: exposes ``start_profile`` / ``stop_profile`` as group calls."""

    def __init__(self, profiler: DistProfiler):
        self.profiler = profiler

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def start_profile(self, **kwargs) -> None:
        self.profiler.start(**kwargs)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def stop_profile(self) -> None:
        self.profiler.stop()
