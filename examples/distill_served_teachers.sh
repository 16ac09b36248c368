#!/usr/bin/env bash
# On-policy distillation from two teachers served on GPUs 6 and 7 (one rollout-server process each); samples are routed to a teacher by
# their data_source. The student trains on GPUs 0-5.
set -euo pipefail
CUDA_VISIBLE_DEVICES=0,1,2,3,4,5,6,7 python -m torch.distributed.run --nnodes=1 --nproc-per-node 6 --master-addr 127.0.0.1 --master-port 29500 \
  -m verl_b200.trainer.main_ppo algorithm.adv_estimator=grpo data.train_files="$TRAIN" data.val_files="$VAL" data.train_batch_size=192 \
  actor_rollout_ref.model.path="$STUDENT" actor_rollout_ref.rollout.n=4 trainer.n_gpus_per_node=6 \
  actor_rollout_ref.distillation.enable=true actor_rollout_ref.distillation.teacher_mode=server actor_rollout_ref.distillation.topk=32 \
  actor_rollout_ref.distillation.teacher_key=data_source "actor_rollout_ref.distillation.teacher_devices=[6,7]" \
  "+actor_rollout_ref.distillation.teacher_models.openai/gsm8k={model_path: $MATH_TEACHER, num_replicas: 1}" \
  "+actor_rollout_ref.distillation.teacher_models.codeforces={model_path: $CODE_TEACHER, num_replicas: 1}" "$@"
