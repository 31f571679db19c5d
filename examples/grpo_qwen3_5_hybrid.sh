#!/usr/bin/env bash
# GRPO on a Qwen3.5-style hybrid stack: three Gated-DeltaNet layers per gated softmax-attention layer, partial rotary,
# zero-centred norms.  Trainer and rollout engine run the linear-attention layers as PyTorch statements (one rank per
# model replica / engine); the engine keeps a convolution window and a recurrent matrix per request.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3.5-9b --colocate --advantage-estimator grpo --apply-layernorm-1p \
  --rollout-batch-size 64 --n-samples-per-prompt 8 --global-batch-size 512 --rollout-max-response-len 1024 \
  --use-dynamic-batch-size --max-tokens-per-gpu 8192 --lr 1e-6 --num-rollout 100 \
  "$@"
