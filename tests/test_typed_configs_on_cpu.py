import pytest

from verl_b200.utils.config import load_config
from verl_b200.workers.config import ActorConfig, AlgoConfig, FSDPActorConfig, HFModelConfig, McoreActorConfig, RolloutConfig, from_config


def test_typed_views_of_the_default_yaml():
    cfg = load_config("ppo_trainer", ["actor_rollout_ref.model.preset=tiny-qwen2", "data.max_prompt_length=64", "data.max_response_length=32"])
    ar = cfg.actor_rollout_ref
    actor = from_config(FSDPActorConfig, ar.actor)
    assert actor.optim.lr == ar.actor.optim.lr and actor["clip_ratio"] == 0.2 and actor.fsdp_config.fsdp_size == -1
    ro = from_config(RolloutConfig, ar.rollout)
    assert ro.prompt_length == 64 and ro.val_kwargs.do_sample is False and ro.multi_turn.format == "hermes" and ro.agent.num_workers == 8
    assert from_config(HFModelConfig, ar.model).preset == "tiny-qwen2"
    algo = from_config(AlgoConfig, cfg.algorithm)
    assert algo.kl_ctrl.type in ("fixed", "adaptive") and dict(algo)["gamma"] == 1.0
    assert from_config(McoreActorConfig, ar.actor, strategy="megatron").megatron.tensor_model_parallel_size == 1


def test_validation_and_immutability():
    with pytest.raises(ValueError):
        ActorConfig(ppo_micro_batch_size=4, ppo_micro_batch_size_per_gpu=2)
    with pytest.raises(ValueError):
        HFModelConfig().validate()
    with pytest.raises(ValueError):
        RolloutConfig(quantization="int3")
    a = ActorConfig(ppo_mini_batch_size=64, ppo_micro_batch_size_per_gpu=3)
    with pytest.raises(ValueError):
        a.validate(n_gpus=8, train_batch_size=32)
    with pytest.raises(ValueError):
        a.validate(n_gpus=8, train_batch_size=128)      # 64/8 = 8 per GPU is not a multiple of 3
    a.ppo_mini_batch_size = 48                           # listed as mutable
    with pytest.raises(Exception):
        a.clip_ratio = 0.3


def test_every_yaml_key_has_a_typed_field_and_the_tree_instantiates():
    """The group files and the dataclasses cannot drift apart: every key of a composed section is a field of the class its
    ``_target_`` names, for both engine families; the composed tree converts section by section."""
    import dataclasses

    from verl_b200.trainer.config import AlgoConfig, DataConfig, TrainerConfig
    from verl_b200.utils.config import load_config, omega_conf_to_dataclass
    from verl_b200.workers.config import (FSDPActorConfig, FSDPCriticConfig, HFModelConfig, McoreActorConfig, McoreCriticConfig, RewardConfig,
                                          RolloutConfig, from_config)

    def check(cls, node, path):
        names = {f.name for f in dataclasses.fields(cls)}
        extra = [k for k in node.keys() if k not in names and k != "_target_"]
        assert not extra, f"{path}: yaml keys without a field in {cls.__name__}: {extra}"
        obj = from_config(cls, node)
        for f in dataclasses.fields(cls):
            sub = f.metadata.get("cls")
            if sub is not None and f.name in node and node[f.name] is not None:
                check(sub, node[f.name], f"{path}.{f.name}")
        return obj

    for engine, actor_cls, critic_cls in (("dp", FSDPActorConfig, FSDPCriticConfig), ("megatron", McoreActorConfig, McoreCriticConfig)):
        c = load_config("ppo_trainer", [f"model_engine={engine}", "actor_rollout_ref.rollout.n=4"])
        a = c.actor_rollout_ref
        actor = check(actor_cls, a.actor, "actor")
        check(actor_cls, a.ref, "ref")
        critic = check(critic_cls, c.critic, "critic")
        ro = check(RolloutConfig, a.rollout, "rollout")
        check(HFModelConfig, a.model, "model")
        check(RewardConfig, c.reward, "reward")
        algo = check(AlgoConfig, c.algorithm, "algorithm")
        check(TrainerConfig, c.trainer, "trainer")
        check(DataConfig, c.data, "data")
        assert actor.rollout_n == 4 and critic.rollout_n == 4 and ro.n == 4 and algo.rollout_correction.loss_type == "ppo_clip"
        assert actor.checkpoint.load_contents == ["model", "optimizer", "extra"] and ro.replicas(8) == 8
        built = omega_conf_to_dataclass(a.actor)                     # through `_target_`
        assert type(built) is actor_cls and built.optim.lr == 1e-6
    with pytest.raises(ValueError):
        from_config(RolloutConfig, {"name": "nope"})
    with pytest.raises(ValueError):
        from_config(RolloutConfig, {"quantization": "int3"})
    with pytest.raises(ValueError):
        from_config(McoreActorConfig, {"megatron": {"virtual_pipeline_model_parallel_size": 2}})
