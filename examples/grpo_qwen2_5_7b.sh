#!/usr/bin/env bash
# GRPO, Qwen2.5-7B, sharded-DP actor + reference colocated with rollout replicas of 2 GPUs, 256 prompts x 8 samples.
# Usage: MODEL=/models/Qwen2.5-7B-Instruct TRAIN=gsm8k/train.parquet VAL=gsm8k/test.parquet NGPU=8 bash examples/grpo_qwen2_5_7b.sh
set -euo pipefail
NGPU=${NGPU:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=grpo data.train_files="$TRAIN" data.val_files="$VAL" data.train_batch_size=256 \
  data.max_prompt_length=512 data.max_response_length=1024 \
  actor_rollout_ref.model.path="$MODEL" actor_rollout_ref.model.enable_gradient_checkpointing=false \
  actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=64 \
  actor_rollout_ref.actor.use_dynamic_bsz=true actor_rollout_ref.actor.ppo_max_token_len_per_gpu=8192 \
  actor_rollout_ref.actor.use_kl_loss=true actor_rollout_ref.actor.kl_loss_coef=0.001 actor_rollout_ref.actor.kl_loss_type=low_var_kl \
  actor_rollout_ref.rollout.n=8 actor_rollout_ref.rollout.tensor_model_parallel_size=2 actor_rollout_ref.rollout.gpu_memory_utilization=0.3 \
  actor_rollout_ref.rollout.log_prob_use_dynamic_bsz=true actor_rollout_ref.ref.log_prob_use_dynamic_bsz=true \
  trainer.total_epochs=15 trainer.save_freq=20 trainer.test_freq=5 trainer.logger='[console,file]' "$@"
