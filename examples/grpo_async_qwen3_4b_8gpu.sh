#!/usr/bin/env bash
# Fully-asynchronous GRPO: rollout, old-policy / reference forward and training run as concurrent roles; a rollout
# may be at most --max-staleness weight versions behind the trainer.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3-4b --fully-async --max-staleness 1 --advantage-estimator grpo \
  --rollout-batch-size 64 --n-samples-per-prompt 8 --global-batch-size 512 \
  --rollout-max-response-len 2048 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  --eps-clip 0.2 --use-tis --lr 1e-6 --num-rollout 200 \
  "$@"
