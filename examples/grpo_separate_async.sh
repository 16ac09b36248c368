#!/usr/bin/env bash
# Separate-pool asynchronous GRPO: GPUs 0-3 train (sharded data parallel), GPUs 4-7 run standalone rollout servers. Prompts
# stream to the servers over HTTP, weights are pushed after every update through a CUDA IPC export buffer, trajectories may be
# up to two policy versions old.
set -euo pipefail
CUDA_DEVICE_ORDER=PCI_BUS_ID python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29500 \
  -m verl_b200.trainer.main_ppo trainer.use_v1=true trainer.trainer_mode=separate_async "+trainer.v1.rollout_devices=[4,5,6,7]" +trainer.v1.max_off_policy_threshold=2 \
  +trainer.v1.async_warmup_batches=1 algorithm.adv_estimator=grpo data.train_files="$TRAIN" data.val_files="$VAL" \
  data.train_batch_size=128 actor_rollout_ref.model.path="$MODEL" actor_rollout_ref.rollout.mode=async actor_rollout_ref.rollout.n=8 \
  algorithm.rollout_correction.rollout_is=token "$@"
