#!/usr/bin/env bash
# Supervised fine-tuning.  sft.jsonl rows: {"messages": [...]} or {"prompt": "...", "response": "..."}; only the
# assistant turns carry loss.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3-4b --loss-type sft_loss --prompt-data sft.jsonl \
  --global-batch-size 256 --use-dynamic-batch-size --max-tokens-per-gpu 16384 \
  --lr 1e-5 --lr-decay-style cosine --lr-warmup-iters 20 --num-rollout 500 --save ckpt/qwen3-4b-sft \
  "$@"
