#!/usr/bin/env bash
# GRPO on a policy with a multi-token-prediction (MTP) block: the block is trained next to the policy
# (--enable-mtp-training) and drafts for the rollout engine (speculative decoding: an accepted proposal yields two
# tokens per pass over the weights; the samples stay exact policy samples).  Tiny preset: runs on a CPU.
set -euo pipefail
python -m relax_b200.entrypoints.train \
  --model-name tiny --colocate --advantage-estimator grpo \
  --rollout-batch-size 4 --n-samples-per-prompt 4 --global-batch-size 16 \
  --rollout-max-response-len 16 --num-rollout 3 --lr 1e-4 --rm-type token_sum_parity \
  --mtp-num-layers 1 --enable-mtp-training --mtp-loss-scaling-factor 0.3 \
  --sglang-speculative-algorithm EAGLE --sglang-speculative-num-steps 2 \
  --sglang-speculative-eagle-topk 1 --sglang-speculative-num-draft-tokens 3 \
  "$@"
