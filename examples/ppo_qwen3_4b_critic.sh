#!/usr/bin/env bash
# PPO with a learned critic (GAE): the value model shares the actor's ranks; the first rollouts train the critic alone.
set -euo pipefail
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
  -m relax_b200.entrypoints.train \
  --model-name qwen3-4b --colocate --advantage-estimator ppo --gamma 1.0 --lambd 0.95 --num-critic-only-steps 2 \
  --tensor-model-parallel-size 2 --rollout-num-gpus-per-engine 2 \
  --rollout-batch-size 64 --n-samples-per-prompt 4 --global-batch-size 256 --rollout-max-response-len 2048 \
  --use-dynamic-batch-size --max-tokens-per-gpu 16384 --eps-clip 0.2 --kl-coef 0.001 --lr 1e-6 --critic-lr 5e-6 \
  --offload-rollout --num-rollout 100 \
  "$@"
