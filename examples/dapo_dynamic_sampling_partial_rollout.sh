#!/usr/bin/env bash
# DAPO-style dynamic sampling with partial rollout: groups whose rewards are all equal are dropped, 2x the batch is in
# flight, generation stops as soon as the batch is full, and the aborted groups continue in the next step with the tokens
# of the older policy masked out of the loss.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3-8b --colocate --advantage-estimator grpo --tensor-model-parallel-size 2 --rollout-num-gpus-per-engine 2 \
  --rollout-batch-size 128 --over-sampling-batch-size 256 --n-samples-per-prompt 8 --global-batch-size 1024 \
  --dynamic-sampling-filter-path relax_b200.rollout.filters:check_reward_nonzero_std \
  --partial-rollout --mask-offpolicy-in-partial-rollout --partial-rollout-max-aborted-count 4 \
  --rollout-max-response-len 4096 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  --eps-clip 0.2 --eps-clip-high 0.28 --lr 1e-6 --offload-rollout --num-rollout 100 \
  "$@"
