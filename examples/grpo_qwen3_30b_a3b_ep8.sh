#!/usr/bin/env bash
# GRPO on a Qwen3-30B-A3B-architecture mixture-of-experts model, 8 GPUs: experts spread over all ranks (16 per rank, token dispatch and
# combine inside the grouped expert GEMMs over NVLink), block-scaled fp8 rollout weights, and router replay of the rollout's expert
# choices into training (R3).
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=grpo data.train_files="$TRAIN" data.val_files="$VAL" data.train_batch_size=128 data.max_prompt_length=1024 \
  data.max_response_length=2048 actor_rollout_ref.model.path="$MODEL" actor_rollout_ref.rollout.n=8 \
  actor_rollout_ref.actor.strategy=megatron actor_rollout_ref.actor.megatron.expert_model_parallel_size=8 \
  actor_rollout_ref.ref.strategy=megatron actor_rollout_ref.ref.megatron.expert_model_parallel_size=8 \
  actor_rollout_ref.rollout.quantization=fp8_block actor_rollout_ref.actor.router_replay.mode=R3 "$@"
