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
        HFModelConfig()
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
