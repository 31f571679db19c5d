#!/usr/bin/env bash
# Sequence classification fine-tuning: a class head on the last token, rows {"prompt": text, "label": id}; for multi-label
# data pass --problem-type multi_label_classification with rows whose label is a list of ids.
set -euo pipefail
python -m relax_b200.entrypoints.train \
  --model-name qwen3-0.6b --loss-type seq_cls_loss --num-labels 4 --prompt-data data/cls_train.jsonl --label-key label \
  --global-batch-size 64 --max-tokens-per-gpu 16384 --lr 2e-5 --num-rollout 500 --save ckpt/cls --save-interval 100 \
  "$@"
