#!/usr/bin/env bash
# GRPO on a GLM-4 dense model (sandwich norms, half rotary, q/k/v bias) - trainer and rollout engine both serve the
# family; weights come from the Hugging Face checkpoint.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name glm4-9b --hf-checkpoint models/GLM-4-9B-0414 --colocate --advantage-estimator grpo \
  --tensor-model-parallel-size 2 --rollout-num-gpus-per-engine 2 \
  --rollout-batch-size 64 --n-samples-per-prompt 8 --global-batch-size 512 --rollout-max-response-len 2048 \
  --use-dynamic-batch-size --max-tokens-per-gpu 16384 --use-kl-loss --kl-loss-coef 0.001 --lr 1e-6 --num-rollout 200 \
  "$@"
