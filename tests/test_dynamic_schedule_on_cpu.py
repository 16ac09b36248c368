"""Lending policies and the resource controller, without any engine (a fake lender records the transitions)."""

import pytest

from verl_b200.experimental.fully_async_policy.dynamic_schedule import (
    DefaultDynamicSchedulePolicy, DynamicResourceController, DynamicScheduleContext, DynamicSchedulePolicyBase, ResourceState,
    build_policy, register_policy, registered_policies)


def ctx(generated=0, expected=0, waits=(), wait_samples=(), required=8, sync=4, act=0.0, deact=0.0):
    c = DynamicScheduleContext(required_samples=required, trigger_parameter_sync_step=sync, total_generated_samples=generated,
                               expected_samples=expected, buffer_samples=64, step_wait_times=list(waits), step_wait_samples=list(wait_samples))
    c.last_activate_duration_s, c.last_deactivate_duration_s = act, deact
    return c


class FakeLender:
    def __init__(self):
        self.calls = []

    def activate(self):
        self.calls.append("activate")

    def deactivate(self):
        self.calls.append("deactivate")

    def rebalance(self):
        self.calls.append("rebalance")
        return {"cleared_entries": 0}


def test_registry_and_context():
    assert {"default", "fixed_ratio", "static_fully_async"} <= set(registered_policies())
    with pytest.raises(KeyError, match="Unknown dynamic scheduling policy"):
        build_policy("nope")
    with pytest.raises(TypeError):
        register_policy("bad")(dict)
    c = ctx(generated=40, expected=32)
    assert c.step_required_samples == 32 and c.surplus == 8

    @register_policy("always_keep")
    class Keep(DynamicSchedulePolicyBase):
        def should_deactivate(self, g, active, c):
            return False

        def deactivate_wait_samples(self, c):
            return 0

        def should_activate_after_step(self, g, active, c):
            return True

    assert isinstance(build_policy("always_keep"), Keep)


def test_default_policy_ratio_moves_with_real_waits_only():
    p = build_policy("default", deactivate_ratio=0.3)
    assert p.deactivate_wait_samples(ctx()) == int(32 * 0.3)
    p.update_after_step(1, ctx(waits=[2.0], wait_samples=[16]))          # half a cycle had to be waited for: step capped at 0.10
    assert p.deactivate_ratio == pytest.approx(0.40)
    p.update_after_step(2, ctx(waits=[0.5], wait_samples=[1], required=25))    # a tiny shortfall (1 %) still moves by the minimum step
    assert p.deactivate_ratio == pytest.approx(0.42)
    p.update_after_step(3, ctx())                                       # served from backlog: take the engines back earlier
    assert p.deactivate_ratio == pytest.approx(0.40)
    p.update_after_step(0, ctx(waits=[9.0], wait_samples=[30]))          # step 0 is the initial sync: no adaptation
    assert p.deactivate_ratio == pytest.approx(0.40)
    for _ in range(100):
        p.update_after_step(5, ctx())
    assert p.deactivate_ratio == pytest.approx(p.min_ratio)
    for _ in range(100):
        p.update_after_step(5, ctx(waits=[1.0], wait_samples=[32]))
    assert p.deactivate_ratio == 1.0


def test_default_policy_activation_needs_a_gap_and_a_net_benefit():
    p = DefaultDynamicSchedulePolicy(deactivate_ratio=0.5)
    # threshold 16 samples; 20 already buffered: nothing to gain
    assert not p.should_activate_after_step(1, False, ctx(generated=52, expected=32))
    # gap of 12 with no rate seen yet: the pessimistic 1000 s/sample makes lending look worth it
    assert p.should_activate_after_step(1, False, ctx(generated=36, expected=32))
    # measured: 0.1 s per sample -> 1.2 s to gain, default switch cost 10 s -> stay
    assert not p.should_activate_after_step(2, False, ctx(generated=36, expected=32, waits=[1.6], wait_samples=[16]))
    assert p.last_decision["switch_cost_s"] == 10.0 and p.last_decision["expected_benefit_s"] == pytest.approx(1.2)
    # once switches are timed (0.2 s + 0.3 s), the same gap pays; a cycle without waits keeps the last rate estimate
    p.update_after_step(3, ctx(act=0.2, deact=0.3))
    assert p.switch_cost() == pytest.approx(0.5)
    assert p.should_activate_after_step(3, False, ctx(generated=36, expected=32))
    # rolling window of three pairs
    for pair in (1.0, 2.0, 3.0):
        p.update_after_step(4, ctx(act=pair, deact=0.0))
    assert p.switch_cost() == pytest.approx(2.0)


def test_only_hybrid_waits_for_the_whole_cycle_and_always_lends_again():
    for name in ("default", "fixed_ratio"):
        p = build_policy(name, deactivate_ratio=0.2, only_hybrid=True)
        assert p.deactivate_ratio == 1.0 and p.deactivate_wait_samples(ctx()) == 32
        assert p.should_activate_after_step(3, False, ctx(generated=999, expected=0))
        p.update_after_step(3, ctx(waits=[5.0], wait_samples=[10]))
        assert p.deactivate_ratio == 1.0


def test_fixed_and_static_policies():
    f = build_policy("fixed_ratio", deactivate_ratio=0.25)
    f.update_after_step(1, ctx(waits=[3.0], wait_samples=[20]))
    assert f.deactivate_ratio == 0.25 and f.deactivate_wait_samples(ctx()) == 8
    assert f.should_activate_after_step(1, False, ctx(generated=39, expected=32)) and not f.should_activate_after_step(1, False, ctx(generated=40, expected=32))
    s = build_policy("static_fully_async")
    assert s.should_deactivate(1, True, ctx()) and s.deactivate_wait_samples(ctx()) == 0 and not s.should_activate_after_step(1, False, ctx())
    with pytest.raises(ValueError):
        build_policy("fixed_ratio", deactivate_ratio=0.0)


def test_controller_state_machine_and_order_of_calls():
    lender = FakeLender()
    c = DynamicResourceController(lender, num_standalone_replicas=2, num_hybrid_replicas=4, policy="fixed_ratio", policy_kwargs={"deactivate_ratio": 0.5})
    assert c.state is ResourceState.STANDALONE_ONLY and not c.only_hybrid
    assert c.wait_threshold(1, ctx()) is None                                  # nothing lent, nothing to take back
    assert not c.before_training(1, ctx(), buffered=lambda: 99)
    m = c.after_weight_sync(1, ctx(generated=34, expected=32))
    assert lender.calls == ["activate", "rebalance"] and c.is_hybrid_active and m["dynamic_schedule/want_activate"] == 1.0
    assert not c.activate(1)                                                   # idempotent
    waited = []
    assert c.wait_threshold(2, ctx()) == 16
    assert not c.before_training(2, ctx(), buffered=lambda: 3)                 # below the threshold and nobody to wait with
    assert c.before_training(2, ctx(), buffered=lambda: 3, wait=waited.append) and waited == [16]
    assert lender.calls[-1] == "deactivate" and c.state is ResourceState.STANDALONE_ONLY and c.deactivate_count == 1
    m = c.after_weight_sync(2, ctx(generated=34, expected=32), more_steps=False)      # last step: nothing to lend for
    assert m["dynamic_schedule/want_activate"] == 0.0 and lender.calls.count("activate") == 1
    # a controller without hybrid engines never switches; one without a pool builds an only-hybrid policy
    assert not DynamicResourceController(FakeLender(), 2, 0, policy="default").activate(1)
    assert DynamicResourceController(FakeLender(), 0, 4).policy.deactivate_ratio == 1.0
