#!/usr/bin/env bash
# Vision-language GRPO: prompts with images (JSONL rows {"prompt": "... <|image_pad|> ...", "image": "path.png", "label": ...}).
# The tower embeds the patches at prefill inside the rollout engine and inside every training micro-batch; the freeze
# switches keep the tower fixed and train the projection + language model.
set -euo pipefail
python -m relax_b200.entrypoints.train \
  --model-name qwen3-vl-8b --colocate --advantage-estimator grpo \
  --prompt-data data/vl_train.jsonl --input-key prompt --label-key label --multimodal-keys '{"image": "image"}' \
  --hf-checkpoint models/Qwen3-VL-8B --apply-chat-template --freeze-vision-model \
  --rollout-batch-size 32 --n-samples-per-prompt 8 --global-batch-size 256 \
  --rollout-max-prompt-len 1024 --rollout-max-response-len 1024 \
  --use-dynamic-batch-size --max-tokens-per-gpu 8192 --eps-clip 0.2 --lr 1e-6 --num-rollout 100 \
  "$@"
