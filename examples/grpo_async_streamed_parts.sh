#!/usr/bin/env bash
# Fully-asynchronous GRPO in which the trainer does not wait for whole rollout batches: the engines publish finished
# prompt groups in four parts per rollout and the trainer runs its forward-only passes (reference and old-policy
# log-probs) on each part while the rest is still being generated.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3-4b --fully-async --max-staleness 1 --num-iters-per-train-update 4 --advantage-estimator grpo \
  --resource '{"actor": [1, 4], "rollout": [1, 4]}' --tensor-model-parallel-size 2 --rollout-num-gpus-per-engine 2 \
  --rollout-batch-size 64 --n-samples-per-prompt 8 --global-batch-size 512 \
  --rollout-max-response-len 2048 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  --use-kl-loss --kl-loss-coef 0.001 --lr 1e-6 --num-rollout 200 \
  "$@"
