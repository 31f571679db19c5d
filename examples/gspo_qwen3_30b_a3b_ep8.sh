#!/usr/bin/env bash
# Mixture-of-experts GSPO on one 8 x B200 node: trainer TP1 x EP8 (experts split over all ranks, one grouped tcgen05 GEMM
# per projection for the local experts), one EP8 rollout engine on the same GPUs, sequence-level ratio clip 3e-4 / 4e-4.
# --use-rollout-routing-replay makes the trainer replay the experts the engine chose for every position (R3).
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3-30b-a3b --colocate --advantage-estimator gspo \
  --expert-model-parallel-size 8 --sglang-ep-size 8 --rollout-num-gpus-per-engine 8 \
  --rollout-batch-size 64 --n-samples-per-prompt 8 --global-batch-size 512 \
  --rollout-max-prompt-len 1024 --rollout-max-response-len 4096 \
  --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  --eps-clip 3e-4 --eps-clip-high 4e-4 --use-rollout-routing-replay \
  --lr 1e-6 --clip-grad 1.0 --offload-rollout --num-rollout 100 \
  "$@"
