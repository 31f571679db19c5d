#!/usr/bin/env bash
# GRPO on rollouts produced by an external agent program: every sample starts one agent process, which talks to the
# policy through the OpenAI-compatible endpoint and reports a reward when it exits.  Tiny preset, runs on a CPU.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
PROMPTS="$(mktemp)"
for i in 0 1 2 3; do echo "{\"prompt\": \"task $i\", \"label\": null}"; done > "$PROMPTS"
python -m relax_b200.entrypoints.train \
  --model-name tiny --colocate --advantage-estimator grpo \
  --rollout-batch-size 4 --n-samples-per-prompt 2 --global-batch-size 8 \
  --rollout-max-response-len 8 --rollout-max-prompt-len 256 --num-rollout 2 --lr 1e-4 \
  --prompt-data "$PROMPTS" --input-key prompt \
  --use-agentic-rollout --agent-command "python echo_agent.py" --agent-cwd "$HERE/agent_command" \
  --agent-timeout 300 --agentic-concurrency 8 --agentic-program-admission \
  "$@"
