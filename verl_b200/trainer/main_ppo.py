"""``python -m verl_b200.trainer.main_ppo key=value ...`` — PPO / GRPO training entry point.

Overrides use the reference's Hydra syntax (``a.b=1``, ``+a.b=1``, ``~a.b``); ``--config-name`` / ``--config-path`` pick
another yaml. Launch under ``torchrun`` for multi-GPU (``trainer.worker_backend=spmd``, the default) or run a single
controller that spawns its own workers (``trainer.worker_backend=process``).
Parity target: ``verl/trainer/main_ppo.py:34-192``.
"""

from __future__ import annotations

import os
import sys

from verl_b200.utils.config import load_config, validate_config


def _load_tokenizer(path):
    if not path or not os.path.isdir(os.path.expanduser(path)):
        return None
    try:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(os.path.expanduser(path))
        if tok.pad_token_id is None:
            tok.pad_token = tok.eos_token
        return tok
    except Exception as e:  # noqa: BLE001
        print(f"no tokenizer loaded from {path}: {e}")
        return None


def run_ppo(config):
    from verl_b200.trainer.ppo.ppo_trainer import PPOTrainer
    from verl_b200.trainer.ppo.reward import load_reward_manager

    from verl_b200.trainer.constants_ppo import apply_worker_runtime_env

    apply_worker_runtime_env(config)       # before any worker process or process group exists
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if config.trainer.get("worker_backend", "spmd") == "spmd":
        config.trainer["n_gpus_per_node"] = max(1, world // int(config.trainer.get("nnodes", 1)))
    trainer_probe_critic = config.critic.get("enable")
    use_critic = trainer_probe_critic if trainer_probe_critic is not None else config.algorithm.adv_estimator == "gae"
    use_ref = bool(config.algorithm.get("use_kl_in_reward", False)) or bool(config.actor_rollout_ref.actor.get("use_kl_loss", False))
    validate_config(config, use_reference_policy=use_ref, use_critic=use_critic)
    tokenizer = _load_tokenizer(config.data.get("tokenizer") or config.actor_rollout_ref.model.get("path"))
    reward_fn = load_reward_manager(config, tokenizer, num_examine=0)
    val_reward_fn = load_reward_manager(config, tokenizer, num_examine=1)
    v1 = config.trainer.get("trainer_mode", "sync") if config.trainer.get("use_v1", False) else None
    if v1:
        # v1 family (generation decoupled through the TransferQueue): sync | colocate_async | separate_async
        from verl_b200.trainer.ppo.v1 import get_trainer_cls

        trainer = get_trainer_cls(str(v1))(config, tokenizer=tokenizer, reward_fn=reward_fn, val_reward_fn=val_reward_fn)
        trainer.init()
        trainer.fit()
        return trainer
    trainer = PPOTrainer(config, tokenizer=tokenizer, reward_fn=reward_fn, val_reward_fn=val_reward_fn)
    trainer.init_workers()
    trainer.fit()
    return trainer


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    name, cdir, overrides = "ppo_trainer", None, []
    i = 0
    while i < len(argv):
        a = argv[i]
        if a in ("--config-name", "-cn"):
            name, i = argv[i + 1], i + 2
        elif a.startswith("--config-name="):
            name, i = a.split("=", 1)[1], i + 1
        elif a in ("--config-path", "-cp"):
            cdir, i = argv[i + 1], i + 2
        elif a.startswith("--config-path="):
            cdir, i = a.split("=", 1)[1], i + 1
        else:
            overrides.append(a)
            i += 1
    config = load_config(name, overrides, config_dir=cdir)
    return run_ppo(config)


if __name__ == "__main__":
    main()
