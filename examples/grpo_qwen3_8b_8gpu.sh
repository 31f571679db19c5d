#!/usr/bin/env bash
# Colocated GRPO on one 8 x B200 node: trainer TP2 x DP4 with the distributed optimizer, four TP2 rollout engines on
# the same GPUs, weights synchronised every step.  Random-init weights unless --load / --hf-checkpoint is given.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3-8b --colocate --advantage-estimator grpo \
  --tensor-model-parallel-size 2 --rollout-num-gpus-per-engine 2 \
  --rollout-batch-size 128 --n-samples-per-prompt 8 --global-batch-size 1024 \
  --rollout-max-response-len 2048 --rollout-temperature 1.0 \
  --use-dynamic-batch-size --max-tokens-per-gpu 16384 --recompute-granularity full \
  --eps-clip 0.2 --use-kl-loss --kl-loss-coef 0.001 --kl-loss-type k1 \
  --lr 1e-6 --weight-decay 0.1 --adam-beta2 0.98 --clip-grad 1.0 \
  --offload-rollout --num-rollout 100 --save ckpt/qwen3-8b-grpo --save-interval 20 \
  "$@"
