#!/usr/bin/env bash
# Supervised fine-tuning with a held-out split: perplexity every 50 steps, and every 200 steps the current weights
# answer the held-out conversations (an engine next to the trainer; completions under <save>/predict/).
set -euo pipefail
python -m relax_b200.entrypoints.train \
  --model-name qwen3-4b --loss-type sft_loss --prompt-data data/sft/train.jsonl \
  --eval-size 256 --eval-interval 50 --sft-predict-interval 200 --rollout-max-response-len 512 \
  --global-batch-size 64 --use-dynamic-batch-size --max-tokens-per-gpu 16384 --sft-prefetch-buffer-size 256 \
  --lr 1e-5 --num-rollout 2000 --save ckpt/sft-qwen3-4b --save-interval 200 \
  "$@"
