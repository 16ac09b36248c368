#!/usr/bin/env bash
# GRPO with low-rank adapters: only the adapters are trained and sharded; the rollout serves them live on the shared base weights,
# so there is no merged copy and no weight hand-off between the trainer and the rollout.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=grpo data.train_files="$TRAIN" data.val_files="$VAL" data.train_batch_size=256 \
  actor_rollout_ref.model.path="$MODEL" actor_rollout_ref.model.lora_rank=32 actor_rollout_ref.model.lora_alpha=64 \
  actor_rollout_ref.model.target_modules=all-linear actor_rollout_ref.actor.optim.lr=3e-5 actor_rollout_ref.rollout.n=8 "$@"
# afterwards: python -m verl_b200.scripts.merge_lora --base "$MODEL" --checkpoint <ckpt>/global_step_N/actor --out merged/
