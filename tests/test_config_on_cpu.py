import dataclasses

import pytest

from verl_b200.base_config import BaseConfig
from verl_b200.utils.config import Config, apply_overrides, load_config, omega_conf_to_dataclass, validate_config


def test_load_and_override_and_interpolate():
    c = load_config("ppo_trainer", ["data.max_response_length=777", "actor_rollout_ref.actor.ppo_mini_batch_size=32", "+extra.key=[1,2]"])
    assert c.actor_rollout_ref.rollout.response_length == 777
    assert c.critic.ppo_mini_batch_size == 32
    assert c.extra.key == [1, 2]
    assert c.trainer.default_local_dir == "checkpoints/verl_b200_examples/gsm8k"


def test_override_unknown_key_needs_plus():
    with pytest.raises(KeyError):
        load_config("ppo_trainer", ["data.not_a_key=1"])
    c = load_config("ppo_trainer", ["++data.not_a_key=1", "~data.val_files"])
    assert c.data.not_a_key == 1 and "val_files" not in c.data


def test_config_attribute_and_select():
    c = Config({"a": {"b": [{"c": 1}]}})
    assert c.a.b[0].c == 1 and c.select("a.b") == [{"c": 1}] and c.select("a.x.y", 5) == 5
    c.a.z = {"w": 2}
    assert c.a.z.w == 2


def test_validate_config_checks():
    base = ["actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4", "trainer.n_gpus_per_node=2", "data.train_batch_size=8",
            "actor_rollout_ref.actor.ppo_mini_batch_size=8", "algorithm.adv_estimator=grpo"]
    validate_config(load_config("ppo_trainer", base))
    with pytest.raises(ValueError):
        validate_config(load_config("ppo_trainer", [b for b in base if "micro" not in b]))
    with pytest.raises(ValueError):
        validate_config(load_config("ppo_trainer", base + ["actor_rollout_ref.actor.ppo_micro_batch_size=8"]))
    with pytest.raises(AssertionError):
        validate_config(load_config("ppo_trainer", base + ["data.train_batch_size=7", "actor_rollout_ref.actor.ppo_mini_batch_size=7"]))
    with pytest.raises(ValueError):
        validate_config(load_config("ppo_trainer", base + ["actor_rollout_ref.actor.loss_agg_mode=bogus"]))


@dataclasses.dataclass
class _Inner(BaseConfig):
    x: int = 1


@dataclasses.dataclass
class _Outer(BaseConfig):
    _mutable_fields = {"lr"}
    lr: float = 0.1
    name: str = "a"
    inner: object = None


def test_base_config_frozen_and_mapping():
    o = _Outer(lr=0.5)
    o.lr = 1.0
    with pytest.raises(dataclasses.FrozenInstanceError):
        o.name = "b"
    assert o["lr"] == 1.0 and o.get("missing", 3) == 3 and "name" in list(o)


def test_omega_conf_to_dataclass_nested():
    cfg = {"_target_": f"{__name__}._Outer", "lr": 0.3, "inner": {"_target_": f"{__name__}._Inner", "x": 7}, "ignored": 1}
    o = omega_conf_to_dataclass(cfg)
    assert isinstance(o, _Outer) and o.lr == 0.3 and isinstance(o.inner, _Inner) and o.inner.x == 7
    assert omega_conf_to_dataclass({"lr": 2.0}, _Outer).lr == 2.0


def test_apply_overrides_types():
    d = {"a": {"b": 1}}
    apply_overrides(d, ["a.b=2.5", "+a.c=true", "+a.d=null", "+a.e=hello"])
    assert d["a"] == {"b": 2.5, "c": True, "d": None, "e": "hello"}
