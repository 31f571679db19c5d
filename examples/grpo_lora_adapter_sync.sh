#!/usr/bin/env bash
# LoRA GRPO with adapter-mode weight sync: the engine keeps the base weights from the first sync and applies the factors at
# run time, so every later sync moves the factors only (a few MB instead of the whole model).
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3-8b --colocate --advantage-estimator grpo --tensor-model-parallel-size 2 --rollout-num-gpus-per-engine 2 \
  --lora-rank 32 --lora-alpha 64 --lora-dropout 0.05 --lora-adapter-mode \
  --rollout-batch-size 32 --n-samples-per-prompt 8 --global-batch-size 256 --rollout-max-response-len 1024 \
  --use-dynamic-batch-size --max-tokens-per-gpu 16384 --eps-clip 0.2 --lr 1e-5 --num-rollout 100 \
  "$@"
