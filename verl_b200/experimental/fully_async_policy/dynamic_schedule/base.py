"""Pluggable policies for lending the training GPUs to generation, and their registry.

A policy answers four questions for the trainer that owns both a standalone rollout pool and "hybrid" engines colocated with
the training ranks: before training — should the hybrid engines be taken back now, and how many finished samples must be
buffered before that happens; after the weight push — should they be lent again; and how internal parameters move with what
the last cycle measured. All questions receive one ``DynamicScheduleContext``.

Custom policy::

    @register_policy("mine")
    class Mine(DynamicSchedulePolicyBase):
        def should_deactivate(self, global_steps, is_hybrid_active, ctx): ...
        def deactivate_wait_samples(self, ctx): ...
        def should_activate_after_step(self, global_steps, is_hybrid_active, ctx): ...

selected with ``dynamic_schedule_policy: mine``.

Reference: ``verl/experimental/fully_async_policy/dynamic_schedule/base.py:36-174`` (registry, context fields, call order).
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass, field

__all__ = ["DynamicScheduleContext", "DynamicSchedulePolicyBase", "register_policy", "build_policy", "registered_policies"]

_REGISTRY: dict = {}


def register_policy(name: str):
    def deco(cls):
        if not (isinstance(cls, type) and issubclass(cls, DynamicSchedulePolicyBase)):
            raise TypeError(f"{cls!r} is not a DynamicSchedulePolicyBase subclass")
        _REGISTRY[name] = cls
        return cls

    return deco


def registered_policies() -> list[str]:
    return sorted(_REGISTRY)


def build_policy(name: str, **kwargs) -> "DynamicSchedulePolicyBase":
    try:
        cls = _REGISTRY[name]
    except KeyError:
        raise KeyError(f"Unknown dynamic scheduling policy {name!r}. Registered: {registered_policies()}") from None
    return cls(**kwargs)


@dataclass
class DynamicScheduleContext:
    """What a policy sees. Constant over a run: ``required_samples`` (one collection: mini-batch × require_batches) and
    ``trigger_parameter_sync_step`` (collections per weight push); their product ``step_required_samples`` is one push cycle.
    Per cycle: ``total_generated_samples`` (finished since the start), ``expected_samples`` (consumed by training up to this
    push), ``buffer_samples`` (staleness head-room), per-collection ``step_wait_times`` with the matching
    ``step_wait_samples`` (samples that were NOT already queued when the collection began — the only ones whose wait says
    something about the generation rate), ``only_hybrid`` (no standalone pool) and the last switch durations."""

    required_samples: int
    trigger_parameter_sync_step: int
    total_generated_samples: int
    expected_samples: int
    buffer_samples: int
    step_wait_times: list = field(default_factory=list)
    step_wait_samples: list = field(default_factory=list)
    only_hybrid: bool = False
    last_activate_duration_s: float = 0.0
    last_deactivate_duration_s: float = 0.0
    step_required_samples: int = field(init=False)

    def __post_init__(self):
        self.step_required_samples = int(self.required_samples) * int(self.trigger_parameter_sync_step)

    @property
    def surplus(self) -> int:
        """Finished samples that training has not consumed yet."""
        return int(self.total_generated_samples) - int(self.expected_samples)


class DynamicSchedulePolicyBase(ABC):
    """Call order per cycle: ``should_deactivate`` → (if true) ``deactivate_wait_samples`` → training + weight push →
    ``update_after_step`` → ``should_activate_after_step`` → (if true) ``request_rebalance``."""

    rebalancer = None          # set by the controller: a callable that spreads open requests over the enlarged pool

    @abstractmethod
    def should_deactivate(self, global_steps: int, is_hybrid_active: bool, ctx: DynamicScheduleContext) -> bool: ...

    @abstractmethod
    def deactivate_wait_samples(self, ctx: DynamicScheduleContext) -> int: ...

    @abstractmethod
    def should_activate_after_step(self, global_steps: int, is_hybrid_active: bool, ctx: DynamicScheduleContext) -> bool: ...

    def update_after_step(self, global_steps: int, ctx: DynamicScheduleContext) -> None:
        return None

    def request_rebalance(self, global_steps: int, ctx: DynamicScheduleContext):
        if self.rebalancer is None:
            return None
        return self.rebalancer()

    def state(self) -> dict:
        """Numbers worth logging each cycle."""
        return {}
