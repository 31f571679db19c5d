#!/usr/bin/env bash
# Fully-asynchronous GRPO on disjoint GPU pools: ranks 0-3 train (TP2 x DP2), ranks 4-7 are two TP2 rollout engines.
# Batches travel through the queue service, a rollout may run at most --max-staleness steps ahead of the trainer, and
# after every step the trainer ranks store the new weights straight into the engines' parameter buffers over NVLink.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3-4b --fully-async --max-staleness 1 --advantage-estimator grpo \
  --resource '{"actor": [1, 4], "rollout": [1, 4]}' --tensor-model-parallel-size 2 --rollout-num-gpus-per-engine 2 \
  --rollout-batch-size 64 --n-samples-per-prompt 8 --global-batch-size 512 \
  --rollout-max-response-len 2048 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  --eps-clip 0.2 --use-tis --lr 1e-6 --num-rollout 200 \
  "$@"
