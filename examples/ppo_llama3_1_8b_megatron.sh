#!/usr/bin/env bash
# PPO with a critic, Llama-3.1-8B, TP2 x PP2 x DP2 engine on 8 GPUs, rollout replicas of 4 GPUs refreshed every step.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=gae algorithm.gamma=1.0 algorithm.lam=1.0 data.train_files="$TRAIN" data.val_files="$VAL" data.train_batch_size=128 \
  data.max_prompt_length=1024 data.max_response_length=2048 actor_rollout_ref.model.path="$MODEL" critic.model.path="$MODEL" \
  actor_rollout_ref.actor.strategy=megatron actor_rollout_ref.ref.strategy=megatron critic.strategy=megatron \
  actor_rollout_ref.actor.megatron.tensor_model_parallel_size=2 actor_rollout_ref.actor.megatron.pipeline_model_parallel_size=2 \
  actor_rollout_ref.ref.megatron.tensor_model_parallel_size=2 actor_rollout_ref.ref.megatron.pipeline_model_parallel_size=2 \
  critic.megatron.tensor_model_parallel_size=2 critic.megatron.pipeline_model_parallel_size=2 critic.cliprange_value=0.5 \
  actor_rollout_ref.rollout.n=1 actor_rollout_ref.rollout.tensor_model_parallel_size=4 "$@"
