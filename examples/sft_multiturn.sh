#!/usr/bin/env bash
# Supervised fine-tuning on (prompt, response) parquet rows with the same engine as RL.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NGPU:-8}" --master-addr 127.0.0.1 --master-port 29500 -m verl_b200.trainer.sft_trainer \
  data.train_files="$TRAIN" data.train_batch_size=256 data.micro_batch_size_per_gpu=8 data.max_prompt_length=1024 data.max_response_length=1024 \
  model.path="$MODEL" optim.lr=1e-5 trainer.total_epochs=3 trainer.save_freq=200 "$@"
