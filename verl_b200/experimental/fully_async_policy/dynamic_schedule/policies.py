"""The three built-in lending policies.

``default``             take the engines back once ``ratio × cycle`` samples are buffered; the ratio rises when training had
                        to wait for generation and falls when it never did; lending again must pay for its own switch cost.
``fixed_ratio``         the same thresholds with a ratio that never moves and no cost/benefit gate.
``static_fully_async``  never lends: hybrid engines are taken back at once and stay with training (plain fully-async).

Reference: ``verl/experimental/fully_async_policy/dynamic_schedule/{default_policy.py:31-235,fixed_ratio_policy.py:23-89,
static_fully_async_policy.py:20-54}``.
"""

from __future__ import annotations

from collections import deque

from .base import DynamicScheduleContext, DynamicSchedulePolicyBase, register_policy

__all__ = ["DefaultDynamicSchedulePolicy", "FixedRatioDynamicSchedulePolicy", "StaticFullyAsyncPolicy"]


class _RatioPolicy(DynamicSchedulePolicyBase):
    def __init__(self, deactivate_ratio: float = 0.3, only_hybrid: bool = False):
        if not 0.0 < float(deactivate_ratio) <= 1.0:
            raise ValueError(f"deactivate_ratio must be in (0, 1], got {deactivate_ratio}")
        self.only_hybrid = bool(only_hybrid)
        # with no standalone pool nothing generates while training runs: the whole cycle must be buffered first
        self.deactivate_ratio = 1.0 if self.only_hybrid else float(deactivate_ratio)

    def should_deactivate(self, global_steps, is_hybrid_active, ctx):
        return bool(is_hybrid_active)

    def deactivate_wait_samples(self, ctx):
        return int(ctx.step_required_samples * self.deactivate_ratio)

    def gap(self, ctx: DynamicScheduleContext) -> float:
        """Samples still missing before the take-back threshold of the coming cycle is met."""
        return self.deactivate_ratio * ctx.step_required_samples - ctx.surplus

    def state(self):
        return {"deactivate_ratio": self.deactivate_ratio}


@register_policy("fixed_ratio")
class FixedRatioDynamicSchedulePolicy(_RatioPolicy):
    def should_activate_after_step(self, global_steps, is_hybrid_active, ctx):
        return True if self.only_hybrid else self.gap(ctx) > 0


@register_policy("default")
class DefaultDynamicSchedulePolicy(_RatioPolicy):
    default_switch_cost_s = 10.0          # used until one activate + deactivate pair has been timed
    window = 3                            # switch costs averaged
    ratio_up_min, ratio_up_max, ratio_down = 0.02, 0.10, 0.02
    initial_per_sample_time_s = 1000.0    # pessimistic: until a real rate is seen, lending always looks worth it

    def __init__(self, deactivate_ratio: float = 0.3, only_hybrid: bool = False, min_ratio: float = 0.02):
        super().__init__(deactivate_ratio, only_hybrid)
        self.min_ratio = float(min_ratio)
        self._switch_costs: deque = deque(maxlen=self.window)
        self._per_sample_time = self.initial_per_sample_time_s
        self.last_decision: dict = {}

    def switch_cost(self) -> float:
        return sum(self._switch_costs) / len(self._switch_costs) if self._switch_costs else self.default_switch_cost_s

    def per_sample_time(self, ctx) -> float:
        """Seconds of waiting per sample that really had to be generated during the wait; backlog served at once carries no
        rate information, so a cycle without real waits keeps the previous estimate."""
        t, n = sum(ctx.step_wait_times), sum(ctx.step_wait_samples)
        if t > 0 and n > 0:
            self._per_sample_time = t / n
        return self._per_sample_time

    def update_after_step(self, global_steps, ctx):
        if global_steps <= 0 or self.only_hybrid:
            return
        pair = ctx.last_activate_duration_s + ctx.last_deactivate_duration_s
        if pair > 0:
            self._switch_costs.append(pair)
        waited = sum(ctx.step_wait_samples)
        if waited > 0:                     # generation was the bottleneck: keep the engines lent for longer next time
            frac = waited / ctx.step_required_samples if ctx.step_required_samples > 0 else self.ratio_up_max
            self.deactivate_ratio = min(1.0, self.deactivate_ratio + min(self.ratio_up_max, max(self.ratio_up_min, frac)))
        else:                              # training was the bottleneck: take them back earlier
            self.deactivate_ratio = max(self.min_ratio, self.deactivate_ratio - self.ratio_down)

    def should_activate_after_step(self, global_steps, is_hybrid_active, ctx):
        if self.only_hybrid:
            return True
        gap = self.gap(ctx)
        if gap <= 0:
            self.last_decision = {"gap": gap, "activate": False}
            return False
        benefit, cost = gap * self.per_sample_time(ctx), self.switch_cost()
        self.last_decision = {"gap": gap, "expected_benefit_s": benefit, "switch_cost_s": cost, "activate": benefit > cost}
        return benefit > cost

    def state(self):
        return {"deactivate_ratio": self.deactivate_ratio, "switch_cost_s": self.switch_cost(), "per_sample_time_s": self._per_sample_time}


@register_policy("static_fully_async")
class StaticFullyAsyncPolicy(DynamicSchedulePolicyBase):
    def __init__(self, deactivate_ratio: float = 0.3, only_hybrid: bool = False):
        self.deactivate_ratio, self.only_hybrid = float(deactivate_ratio), bool(only_hybrid)

    def should_deactivate(self, global_steps, is_hybrid_active, ctx):
        return bool(is_hybrid_active)

    def deactivate_wait_samples(self, ctx):
        return 0

    def should_activate_after_step(self, global_steps, is_hybrid_active, ctx):
        return False
