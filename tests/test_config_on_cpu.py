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


def test_config_tree_composition_and_reference_style_overrides():
    """The trainer config is composed from group files; an override list written for the reference's tree (the launch
    script of its Qwen3-8B GRPO example, plus group choices) parses unchanged."""
    from verl_b200.scripts.generate_trainer_config import main as gen_main
    from verl_b200.utils.config import load_config

    ov = ["algorithm.adv_estimator=grpo", "algorithm.use_kl_in_reward=False", "data.train_files=['a/train.parquet', 'b/train.parquet']",
          "data.val_files=['a/test.parquet']", "data.train_batch_size=256", "data.max_prompt_length=1024", "data.max_response_length=2048",
          "data.filter_overlong_prompts=True", "data.truncation='error'", "actor_rollout_ref.model.path=/models/Qwen3-8B",
          "actor_rollout_ref.model.use_remove_padding=True", "actor_rollout_ref.model.enable_gradient_checkpointing=True",
          "actor_rollout_ref.actor.optim.lr=1e-6", "actor_rollout_ref.actor.ppo_mini_batch_size=64", "actor_rollout_ref.actor.use_dynamic_bsz=True",
          "actor_rollout_ref.actor.ppo_max_token_len_per_gpu=24576", "actor_rollout_ref.actor.use_kl_loss=True", "actor_rollout_ref.actor.kl_loss_coef=0.001",
          "actor_rollout_ref.actor.kl_loss_type=low_var_kl", "actor_rollout_ref.actor.entropy_coeff=0", "actor_rollout_ref.actor.fsdp_config.param_offload=False",
          "actor_rollout_ref.actor.fsdp_config.optimizer_offload=False", "actor_rollout_ref.rollout.name=vllm", "actor_rollout_ref.rollout.tensor_model_parallel_size=2",
          "actor_rollout_ref.rollout.gpu_memory_utilization=0.6", "actor_rollout_ref.rollout.n=8", "actor_rollout_ref.rollout.log_prob_use_dynamic_bsz=True",
          "actor_rollout_ref.rollout.log_prob_max_token_len_per_gpu=24576", "actor_rollout_ref.ref.log_prob_use_dynamic_bsz=True",
          "actor_rollout_ref.ref.log_prob_max_token_len_per_gpu=24576", "actor_rollout_ref.ref.fsdp_config.param_offload=True", "trainer.balance_batch=True",
          'trainer.logger=["console","wandb"]', "trainer.project_name=p", "trainer.experiment_name=e", "trainer.n_gpus_per_node=8", "trainer.nnodes=1",
          "trainer.save_freq=20", "trainer.test_freq=5", "trainer.total_epochs=15", "ray_kwargs.ray_init.num_cpus=null",
          "+actor_rollout_ref.rollout.engine_kwargs.vllm.attention_backend=flash"]
    c = load_config("ppo_trainer", ov)
    a = c.actor_rollout_ref
    assert c.data.train_files == ["a/train.parquet", "b/train.parquet"] and c.trainer.logger == ["console", "wandb"]
    assert a.actor.fsdp_config.fsdp_size == -1 and a.actor.optim.lr == 1e-6 and a.actor.checkpoint.load_contents == ["model", "optimizer", "extra"]
    assert a.ref.fsdp_config.param_offload is True and a.ref.fsdp_config.forward_only is True and a.ref.strategy == "fsdp"
    assert a.ref.log_prob_max_token_len_per_gpu == 24576 and a.rollout.log_prob_use_dynamic_bsz is True
    assert a.rollout.engine_kwargs.vllm.attention_backend == "flash" and a.rollout.prompt_length == 1024
    assert c.critic.ppo_mini_batch_size == 64 and c.critic.use_dynamic_bsz is True and c.critic.forward_max_token_len_per_gpu == 32768
    assert c.critic.model.value_head is True and c.critic.model.path is None
    assert a.actor.profiler.save_path == "outputs/profile" and a.actor.profiler.tool_config.nsys.discrete is False

    m = load_config("ppo_trainer", ["model_engine=megatron", "actor_rollout_ref.actor.megatron.tensor_model_parallel_size=2",
                                    "actor_rollout_ref.actor.megatron.pipeline_model_parallel_size=2", "critic.megatron.tensor_model_parallel_size=2"])
    assert m.model_engine == "megatron" and m.actor_rollout_ref.actor.strategy == "megatron" and m.critic.strategy == "megatron"
    assert m.actor_rollout_ref.ref.megatron.pipeline_model_parallel_size == 2 and m.actor_rollout_ref.actor.optim.use_distributed_optimizer is True
    one = load_config("ppo_trainer", ["actor@actor_rollout_ref.actor=megatron_actor"])          # one role on the other engine family
    assert one.actor_rollout_ref.actor.strategy == "megatron" and one.critic.strategy == "fsdp"
    aliased = load_config("ppo_trainer", ["critic.fsdp.param_offload=true", "distillation.enabled=true", "reward.reward_manager.name=dapo"])
    assert aliased.critic.fsdp_config.param_offload is True and aliased.actor_rollout_ref.distillation.enable is True and aliased.reward.reward_manager == "dapo"
    sft = load_config("sft_trainer_engine", ["engine=megatron", "optim=megatron", "engine.tensor_model_parallel_size=2"])
    assert sft.engine.tensor_model_parallel_size == 2 and sft.optim.lr == 1e-5 and sft.model.enable_gradient_checkpointing is True
    assert gen_main(["--check"]) == 0                      # the committed composed files are current


def test_every_example_script_parses_against_the_config_tree(monkeypatch):
    """The override lists of ``examples/*.sh`` (the part after ``main_ppo``) must compose with ``ppo_trainer.yaml`` as they are."""
    import glob
    import os
    import shlex

    from verl_b200.utils.config import load_config

    for k in ("TRAIN", "VAL", "MODEL", "STUDENT", "TEACHER", "MATH_TEACHER", "CODE_TEACHER"):
        monkeypatch.setenv(k, f"/data/{k.lower()}")
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
    seen = 0
    for f in sorted(glob.glob(os.path.join(root, "*.sh"))):
        body = " ".join(line.rstrip("\\").strip() for line in open(f).read().splitlines() if not line.startswith("#") and not line.startswith("set "))
        i = body.find("main_ppo")
        if i < 0:
            continue
        args = shlex.split(os.path.expandvars(body[i + len("main_ppo"):].replace('"$@"', "")))
        cfg = load_config("ppo_trainer", args)
        assert cfg.data.train_files == "/data/train", f
        seen += 1
    assert seen >= 10
