#!/usr/bin/env bash
# On-policy distillation on token SETS instead of the sampled token: student and teacher distributions are compared
# on the union of their top-16 ids per position with a Jensen-Shannon divergence (alpha 0.5, tail bin for the rest
# of the mass); the teacher is loaded next to the student (its own snapshot on the training GPUs).
set -euo pipefail
python -m relax_b200.entrypoints.train \
  --model-name qwen3-0.6b --colocate --advantage-estimator grpo --use-opd --opd-teacher-load ckpt/qwen3-8b-teacher \
  --opd-kl-coef 1.0 --opd-token-selection union --opd-log-prob-top-k 16 --opd-kl-type jsd --opd-jsd-alpha 0.5 \
  --opd-norm-mode tail --opd-per-token-clip 10 \
  --rollout-batch-size 32 --n-samples-per-prompt 4 --global-batch-size 128 --rollout-max-response-len 1024 \
  --use-dynamic-batch-size --max-tokens-per-gpu 8192 --lr 1e-6 --num-rollout 100 \
  "$@"
