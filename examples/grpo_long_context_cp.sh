#!/usr/bin/env bash
# Long-context GRPO with context parallelism (K/V all-gather, CP=4): works for any head count, unlike the head-scattering
# Ulysses variant in grpo_long_context_ulysses.sh.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=grpo data.train_files="$TRAIN" data.val_files="$VAL" data.train_batch_size=32 \
  data.max_prompt_length=2048 data.max_response_length=16384 actor_rollout_ref.model.path="$MODEL" \
  +actor_rollout_ref.actor.fsdp_config.context_parallel_size=4 +actor_rollout_ref.ref.fsdp_config.context_parallel_size=4 \
  actor_rollout_ref.actor.use_dynamic_bsz=true actor_rollout_ref.actor.ppo_max_token_len_per_gpu=32768 \
  actor_rollout_ref.rollout.n=8 actor_rollout_ref.rollout.max_model_len=18432 "$@"
