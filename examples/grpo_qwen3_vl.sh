#!/usr/bin/env bash
# GRPO on image (and video-frame) prompts with a Qwen2-VL / Qwen2.5-VL / Qwen3-VL checkpoint: rows carry `images` (and `videos`:
# lists of frame sequences) and mark them with <image> / <video> in the prompt; the tower runs at prefill in the rollout engine and
# inside the training forward, deep-stack features of Qwen3-VL join the decoder's stream in both.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=grpo data.train_files="$TRAIN" data.val_files="$VAL" data.train_batch_size=128 data.image_key=images data.video_key=videos \
  data.image_max_pixels=1003520 data.video_nframes=16 data.max_prompt_length=4096 data.max_response_length=1024 \
  actor_rollout_ref.model.path="$MODEL" actor_rollout_ref.rollout.n=8 actor_rollout_ref.rollout.tensor_model_parallel_size=1 "$@"
