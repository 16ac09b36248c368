#!/usr/bin/env bash
# On-policy distillation: the student samples, a frozen teacher scores its samples (top-32 head), the student minimises the
# forward KL to the teacher's head. Add actor_rollout_ref.distillation.use_policy_loss=true to keep the GRPO loss as well.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=grpo data.train_files="$TRAIN" data.val_files="$VAL" data.train_batch_size=256 \
  actor_rollout_ref.model.path="$STUDENT" actor_rollout_ref.distillation.enable=true actor_rollout_ref.distillation.teacher_model.path="$TEACHER" \
  actor_rollout_ref.distillation.topk=32 actor_rollout_ref.distillation.loss=forward_kl actor_rollout_ref.rollout.n=4 "$@"
