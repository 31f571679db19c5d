#!/usr/bin/env bash
# Capture the advantage and policy-loss stages of rollouts 10 and 11 of a run, then check and re-run the bundle on
# any host (no GPU, no engine): the report names the first record and field that differ.
set -euo pipefail
export RELAX_REPLAY_CAPTURE_DIR=replay-bundles RELAX_REPLAY_CAPTURE_ROLLOUTS=10,11
python -m relax_b200.entrypoints.train \
  --model-name tiny --colocate --advantage-estimator grpo \
  --rollout-batch-size 4 --n-samples-per-prompt 4 --global-batch-size 16 \
  --rollout-max-response-len 16 --num-rollout 12 --lr 1e-4 --rm-type token_sum_parity \
  "$@"
python -m relax_b200.utils.replay validate replay-bundles
python -m relax_b200.utils.replay replay replay-bundles --stage all
