#!/usr/bin/env bash
# Held-out evaluation every 2 steps (mean reward, pass@k, truncation ratio per set), one dump file per rollout step,
# then the viewer on the dumps.  held.jsonl rows: {"prompt": "...", "label": ...}.
set -euo pipefail
python -m relax_b200.entrypoints.train \
  --model-name tiny --colocate --rollout-batch-size 4 --n-samples-per-prompt 4 --global-batch-size 16 \
  --rollout-max-response-len 16 --num-rollout 4 \
  --eval-interval 2 --eval-prompt-data held held.jsonl --n-samples-per-eval-prompt 4 --eval-temperature 0.6 \
  --save-debug-rollout-data dumps/ \
  "$@"
python -m relax_b200.entrypoints.visualize --dir dumps/ --text
# python -m relax_b200.entrypoints.visualize --dir dumps/ --port 8089     # HTML
