"""Profiler configuration (reference: ``verl/utils/profiler/config.py:44-354``)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from verl_b200.base_config import BaseConfig

__all__ = ["ProfilerConfig", "TorchProfilerToolConfig", "TorchMemoryToolConfig", "NsightToolConfig", "PrecisionDebuggerToolConfig"]


@dataclass
class NsightToolConfig(BaseConfig):
    """``discrete``: one report per annotated call instead of one per step; the ``*_nsight_options`` mappings become the
    ``nsys profile`` options of the controller / worker processes (``utils/profiler/nsys.py``)."""

    discrete: bool = False
    controller_nsight_options: Optional[dict] = None
    worker_nsight_options: Optional[dict] = None


@dataclass
class PrecisionDebuggerToolConfig(BaseConfig):
    """Stages to fingerprint (``None`` = all) and whether an unknown stage name is an error."""

    stages: Optional[list] = None
    strict: bool = False


@dataclass
class TorchProfilerToolConfig(BaseConfig):
    step_start: int = -1
    step_end: int = -1
    wait: int = 0
    warmup: int = 0
    active: int = 1
    repeat: int = 1
    with_stack: bool = False
    record_shapes: bool = False


@dataclass
class TorchMemoryToolConfig(BaseConfig):
    trace_alloc_max_entries: int = 100_000
    stack_depth: int = 32


@dataclass
class ProfilerConfig(BaseConfig):
    """``tool`` ∈ {None, "nsys", "torch", "torch_memory"}; ``all_ranks`` or ``ranks`` select who profiles."""

    tool: Optional[str] = None
    enable: bool = False
    all_ranks: bool = False
    ranks: list = field(default_factory=list)
    save_path: str = "outputs/profile"
    tool_config: Optional[dict] = None
    finish_hook_cmd: Optional[str] = None

    def union(self, other: "ProfilerConfig") -> "ProfilerConfig":
        return ProfilerConfig(tool=self.tool or other.tool, enable=self.enable or other.enable, all_ranks=self.all_ranks or other.all_ranks,
                              ranks=sorted(set(self.ranks) | set(other.ranks)), save_path=self.save_path, tool_config=self.tool_config or other.tool_config,
                              finish_hook_cmd=self.finish_hook_cmd or other.finish_hook_cmd)

    def __post_init__(self):
        assert self.tool in (None, "nsys", "torch", "torch_memory", "npu", "precision_debugger"), f"unknown profiler tool {self.tool}"
        assert isinstance(self.ranks, (list, tuple)), "ranks must be a list"
