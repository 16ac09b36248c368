#!/usr/bin/env bash
# Long-context PPO on the TP x PP x CP x DP engine: 2 pipeline ranks x 2 virtual stages each (interleaved 1F1B), zig-zag context
# parallelism over 2 ranks, sequence-parallel tensor parallelism over 2 ranks.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=grpo data.train_files="$TRAIN" data.val_files="$VAL" data.train_batch_size=64 data.max_prompt_length=4096 \
  data.max_response_length=12288 actor_rollout_ref.model.path="$MODEL" actor_rollout_ref.rollout.n=4 \
  actor_rollout_ref.actor.strategy=megatron actor_rollout_ref.ref.strategy=megatron \
  actor_rollout_ref.actor.megatron.tensor_model_parallel_size=2 actor_rollout_ref.actor.megatron.sequence_parallel=true \
  actor_rollout_ref.actor.megatron.pipeline_model_parallel_size=2 actor_rollout_ref.actor.megatron.virtual_pipeline_model_parallel_size=2 \
  actor_rollout_ref.actor.megatron.context_parallel_size=2 actor_rollout_ref.actor.megatron.context_parallel_zigzag=true \
  actor_rollout_ref.ref.megatron.tensor_model_parallel_size=2 actor_rollout_ref.ref.megatron.pipeline_model_parallel_size=2 \
  actor_rollout_ref.ref.megatron.context_parallel_size=2 actor_rollout_ref.rollout.tensor_model_parallel_size=2 "$@"
