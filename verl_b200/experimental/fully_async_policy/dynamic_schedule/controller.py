"""State machine STANDALONE_ONLY ⇄ HYBRID_ACTIVE around a lending policy.

The controller owns no engines. It drives a *lender* — any object with ``activate()`` (push weights to the colocated engines,
wake them, register them with the load balancer), ``deactivate()`` (in this order: stop routing to them, abort what they run so
that clients resume elsewhere, release their KV cache) and optionally ``rebalance()`` — times both transitions, and asks the
policy when to make them.

Reference: ``verl/experimental/fully_async_policy/dynamic_schedule/dynamic_resource_controller.py:50-160``.
"""

from __future__ import annotations

import enum
import time
from typing import Callable, Optional

from .base import DynamicScheduleContext, DynamicSchedulePolicyBase, build_policy

__all__ = ["DynamicResourceController", "ResourceState"]


class ResourceState(enum.Enum):
    STANDALONE_ONLY = "standalone_only"
    HYBRID_ACTIVE = "hybrid_active"


class DynamicResourceController:
    def __init__(self, lender, num_standalone_replicas: int, num_hybrid_replicas: int,
                 policy: Optional[DynamicSchedulePolicyBase | str] = None, policy_kwargs: Optional[dict] = None):
        self.lender = lender
        self.num_standalone, self.num_hybrid = int(num_standalone_replicas), int(num_hybrid_replicas)
        self.only_hybrid = self.num_standalone == 0
        if policy is None or isinstance(policy, str):
            policy = build_policy(policy or "default", only_hybrid=self.only_hybrid, **(policy_kwargs or {}))
        self.policy = policy
        self.policy.rebalancer = getattr(lender, "rebalance", None)
        self.state = ResourceState.STANDALONE_ONLY
        self.activate_count = self.deactivate_count = 0
        self.last_activate_duration_s = self.last_deactivate_duration_s = 0.0
        self.log: list = []

    @property
    def is_hybrid_active(self) -> bool:
        return self.state is ResourceState.HYBRID_ACTIVE

    @property
    def has_hybrid_replicas(self) -> bool:
        return self.num_hybrid > 0

    # ------------------------------------------------------------------ transitions
    def activate(self, global_steps: int) -> bool:
        if not self.has_hybrid_replicas or self.is_hybrid_active:
            return False
        t0 = time.perf_counter()
        self.lender.activate()
        self.last_activate_duration_s = time.perf_counter() - t0
        self.state = ResourceState.HYBRID_ACTIVE
        self.activate_count += 1
        self.log.append(("activate", global_steps))
        return True

    def deactivate(self, global_steps: int) -> bool:
        if not self.is_hybrid_active:
            return False
        t0 = time.perf_counter()
        self.lender.deactivate()
        self.last_deactivate_duration_s = time.perf_counter() - t0
        self.state = ResourceState.STANDALONE_ONLY
        self.deactivate_count += 1
        self.log.append(("deactivate", global_steps))
        return True

    # ------------------------------------------------------------------ policy-driven entry points
    def stamp(self, ctx: DynamicScheduleContext) -> DynamicScheduleContext:
        ctx.only_hybrid = self.only_hybrid
        ctx.last_activate_duration_s, ctx.last_deactivate_duration_s = self.last_activate_duration_s, self.last_deactivate_duration_s
        return ctx

    def wait_threshold(self, global_steps: int, ctx: DynamicScheduleContext) -> Optional[int]:
        """Samples that must be buffered before the engines are taken back, or None when the policy keeps them lent."""
        if not self.policy.should_deactivate(global_steps, self.is_hybrid_active, self.stamp(ctx)):
            return None
        return max(0, int(self.policy.deactivate_wait_samples(ctx)))

    def before_training(self, global_steps: int, ctx: DynamicScheduleContext, buffered: Callable[[], int],
                        wait: Optional[Callable[[int], None]] = None) -> bool:
        """Take the engines back if the policy says so; ``wait(n)`` blocks until ``n`` samples are buffered."""
        need = self.wait_threshold(global_steps, ctx)
        if need is None:
            return False
        if buffered() < need:
            if wait is None:
                return False
            wait(need)
        return self.deactivate(global_steps)

    def after_weight_sync(self, global_steps: int, ctx: DynamicScheduleContext, more_steps: bool = True) -> dict:
        """Adapt the policy, then lend again when it asks for it. Returns metrics."""
        ctx = self.stamp(ctx)
        self.policy.update_after_step(global_steps, ctx)
        want = bool(more_steps) and bool(self.policy.should_activate_after_step(global_steps, self.is_hybrid_active, ctx))
        did = self.activate(global_steps) if want else False
        if did:
            self.policy.request_rebalance(global_steps, ctx)
        m = {f"dynamic_schedule/{k}": float(v) for k, v in self.policy.state().items()}
        m.update({"dynamic_schedule/want_activate": float(want), "dynamic_schedule/hybrid_active": float(self.is_hybrid_active),
                  "dynamic_schedule/activate_count": float(self.activate_count), "dynamic_schedule/deactivate_count": float(self.deactivate_count),
                  "dynamic_schedule/surplus": float(ctx.surplus)})
        return m
