#!/usr/bin/env bash
# On-policy distillation against a remote teacher: start the teacher service on its own GPU, then point the training job at
# it; the student's samples are scored by the teacher before every training step and the reverse KL shapes the advantages.
set -euo pipefail
python -m relax_b200.entrypoints.serve teacher --model-name qwen3-8b --hf-checkpoint models/Qwen3-8B --port 18200 &
TEACHER=$!
trap 'kill $TEACHER' EXIT
python -m relax_b200.entrypoints.train \
  --model-name qwen3-0.6b --colocate --advantage-estimator grpo --opd-type sglang --opd-kl-coef 1.0 \
  --opd-teacher-urls http://127.0.0.1:18200 \
  --rollout-batch-size 32 --n-samples-per-prompt 4 --global-batch-size 128 --rollout-max-response-len 1024 \
  --use-dynamic-batch-size --max-tokens-per-gpu 8192 --lr 1e-6 --num-rollout 100 \
  "$@"
