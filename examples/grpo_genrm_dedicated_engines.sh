#!/usr/bin/env bash
# A generative reward model on GPUs of its own: two grader engine servers are started first, the training job sends
# every finished sample to them (round robin, a server that fails is skipped until it answers again).
set -euo pipefail
for i in 0 1; do
  CUDA_VISIBLE_DEVICES=$((6 + i)) python -m relax_b200.entrypoints.serve engine --model-name qwen3-8b \
    --hf-checkpoint models/Qwen3-8B --port $((18500 + i)) &
done
trap 'kill $(jobs -p)' EXIT
CUDA_VISIBLE_DEVICES=0,1,2,3,4,5 python -m torch.distributed.run --nnodes=1 --nproc-per-node 6 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3-4b --colocate --advantage-estimator grpo --tensor-model-parallel-size 2 --rollout-num-gpus-per-engine 2 \
  --genrm-num-gpus 2 --genrm-engine-addrs 127.0.0.1:18500 127.0.0.1:18501 \
  --prompt-data data/math/train.jsonl --input-key prompt --label-key answer \
  --rollout-batch-size 48 --n-samples-per-prompt 8 --global-batch-size 384 --rollout-max-response-len 2048 \
  --use-dynamic-batch-size --max-tokens-per-gpu 16384 --lr 1e-6 --num-rollout 200 \
  "$@"
