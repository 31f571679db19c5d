#!/usr/bin/env bash
# GRPO on rollout engines that run as their own servers: two are named at start, a third is on standby for the
# autoscaler; the training job checks what they serve, ships its weights to them after every step and exposes
# /scale_out, /scale_in and /engines on the control port (curl -X POST :18400/scale_out -d '{"engine_urls": [...]}').
set -euo pipefail
for port in 18301 18302 18303; do
  python -m relax_b200.entrypoints.serve engine --model-name qwen3-4b --port "$port" &
done
trap 'kill $(jobs -p)' EXIT
cat > /tmp/autoscaler.json <<'JSON'
{"min_engines": 2, "max_engines": 3, "scale_out_cooldown_s": 120, "scale_in_cooldown_s": 600,
 "rules": [{"metric": "queue_depth_per_engine", "threshold": 8, "direction": "above", "for_s": 30},
           {"metric": "kv_cache_utilization", "threshold": 0.2, "direction": "below", "for_s": 600}]}
JSON
python -m relax_b200.entrypoints.train \
  --model-name qwen3-4b --colocate --advantage-estimator grpo \
  --rollout-external --rollout-external-engine-addrs 127.0.0.1:18301 127.0.0.1:18302 \
  --rollout-standby-engine-addrs 127.0.0.1:18303 --elastic-control-port 18400 --autoscaler-config /tmp/autoscaler.json \
  --scale-weight-sync-precheck --scale-out-timeout 600 --scale-in-drain-timeout 120 \
  --rollout-batch-size 32 --n-samples-per-prompt 8 --global-batch-size 256 --rollout-max-response-len 1024 \
  --use-dynamic-batch-size --max-tokens-per-gpu 16384 --lr 1e-6 --num-rollout 100 \
  "$@"
