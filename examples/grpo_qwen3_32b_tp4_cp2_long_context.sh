#!/usr/bin/env bash
# Long-context GRPO, Qwen3-32B shape: trainer TP4 x CP2 (zig-zag context parallelism, peers' K/V staged over NVLink),
# two TP4 rollout engines, 2k-token prompts with up to 16k new tokens, balanced micro-batches.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3-32b --colocate --advantage-estimator grpo \
  --tensor-model-parallel-size 4 --context-parallel-size 2 --rollout-num-gpus-per-engine 4 \
  --rollout-batch-size 32 --n-samples-per-prompt 8 --global-batch-size 256 \
  --rollout-max-prompt-len 2048 --rollout-max-response-len 16384 \
  --use-dynamic-batch-size --max-tokens-per-gpu 20480 --balance-data --recompute-granularity full \
  --eps-clip 0.2 --use-kl-loss --kl-loss-coef 0.001 --lr 1e-6 --offload-rollout --num-rollout 100 \
  "$@"
