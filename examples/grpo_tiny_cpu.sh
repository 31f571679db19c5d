#!/usr/bin/env bash
# The whole colocated loop (rollout engine, rewards, data plane, trainer, weight sync) on the tiny preset; runs on
# a CPU in seconds.
set -euo pipefail
python -m relax_b200.entrypoints.train \
  --model-name tiny --colocate --advantage-estimator grpo \
  --rollout-batch-size 4 --n-samples-per-prompt 4 --global-batch-size 16 \
  --rollout-max-response-len 16 --num-rollout 3 --lr 1e-4 --rm-type token_sum_parity \
  "$@"
