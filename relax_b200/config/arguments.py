"""Command-line surface: flag names, defaults and mode rules of the reference
(relax/utils/arguments.py: groups at :150-2640, three-phase parse :2782-2852,
validation :3230-3971; Megatron-side defaults relax/backends/megatron/arguments.py:
266-351), re-stated as one declarative table.

Parse phases: (1) mode flags (``--colocate / --fully-async / --hybrid``) and
``--resource`` are read first because they decide defaults; (2) rollout-engine
flags are accepted under the reference's ``--sglang-*`` prefix and mapped to the
in-house engine; (3) model/parallel/optimizer flags use Megatron's names.
"""
from __future__ import annotations

import argparse
import json
from typing import Optional, Sequence

ADVANTAGE_ESTIMATORS = ("grpo", "gspo", "sapo", "cispo", "m2po", "rloo", "reinforce_plus_plus",
                        "reinforce_plus_plus_baseline", "ppo", "on_policy_distillation")
LOSS_TYPES = ("policy_loss", "sft_loss", "value_loss", "seq_cls_loss", "custom_loss")


def _b(default=False):
    return {"action": "store_true", "default": default}


# group -> [(flag, kwargs)]
FLAGS: dict[str, list] = {
    "cluster": [
        ("--resource", dict(type=str, default=None, help='JSON {role: [num_serves, num_gpus]}, e.g. {"actor":[1,8],"rollout":[1,8]}')),
        ("--actor-num-nodes", dict(type=int, default=1)), ("--actor-num-gpus-per-node", dict(type=int, default=8)),
        ("--critic-num-nodes", dict(type=int, default=None)), ("--critic-num-gpus-per-node", dict(type=int, default=None)),
        ("--rollout-num-gpus", dict(type=int, default=None)), ("--rollout-num-gpus-per-engine", dict(type=int, default=1)),
        ("--num-gpus-per-node", dict(type=int, default=8)),
        ("--colocate", _b()), ("--fully-async", _b()), ("--hybrid", _b()),
        ("--offload", _b()), ("--offload-train", dict(action="store_true", default=None)),
        ("--offload-rollout", dict(action="store_true", default=None)), ("--selective-offload", _b()),
        ("--max-staleness", dict(type=int, default=0)),
        ("--distributed-backend", dict(type=str, default="nccl")), ("--distributed-timeout-minutes", dict(type=int, default=10)),
        ("--train-backend", dict(type=str, default="native", choices=["native", "megatron"])),
        ("--enable-affinity", _b()), ("--train-env-vars", dict(type=json.loads, default={})),
        ("--train-memory-margin-bytes", dict(type=int, default=1 << 30)),
    ],
    "train": [
        ("--num-rollout", dict(type=int, default=None)), ("--num-epoch", dict(type=int, default=None)),
        ("--global-batch-size", dict(type=int, default=None)), ("--micro-batch-size", dict(type=int, default=1)),
        ("--num-steps-per-rollout", dict(type=int, default=None)), ("--num-iters-per-train-update", dict(type=int, default=1)),
        ("--use-dynamic-batch-size", _b()), ("--use-dynamic-global-batch-size", _b()),
        ("--max-tokens-per-gpu", dict(type=int, default=None)), ("--log-probs-max-tokens-per-gpu", dict(type=int, default=None)),
        ("--log-probs-chunk-size", dict(type=int, default=-1)), ("--balance-data", _b()),
        ("--data-pad-size-multiplier", dict(type=int, default=128)), ("--qkv-format", dict(type=str, default="thd", choices=["thd", "bshd"])),
        ("--recompute-loss-function", _b()), ("--calculate-per-token-loss", _b()),
        ("--true-on-policy-mode", _b()), ("--keep-old-actor", _b()), ("--allgather-cp", _b()),
        ("--update-weights-interval", dict(type=int, default=1)), ("--update-weight-buffer-size", dict(type=int, default=512 * 1024 ** 2)),
        ("--check-weight-update-equal", _b()), ("--disable-weights-backuper", _b()),
        ("--only-train-params-name-list", dict(type=str, nargs="*", default=None)),
        ("--freeze-params-name-list", dict(type=str, nargs="*", default=None)),
        ("--freeze-language-model", _b()), ("--freeze-vision-model", _b()), ("--freeze-vision-projection", _b()),
        ("--debug-rollout-only", _b()), ("--debug-train-only", _b()),
        ("--save-debug-rollout-data", dict(type=str, default=None)), ("--load-debug-rollout-data", dict(type=str, default=None)),
        ("--save-debug-train-data", dict(type=str, default=None)), ("--dump-details", dict(type=str, default=None)),
        ("--start-rollout-id", dict(type=int, default=None)), ("--seed", dict(type=int, default=1234)),
    ],
    "checkpoint": [
        ("--load", dict(type=str, default=None)), ("--save", dict(type=str, default=None)),
        ("--save-interval", dict(type=int, default=None)), ("--hf-checkpoint", dict(type=str, default=None)),
        ("--ref-load", dict(type=str, default=None)), ("--ref-ckpt-step", dict(type=int, default=None)),
        ("--skip-hf-validate", _b()),       # do not compare the model shape with the config.json under --hf-checkpoint
        ("--ref-update-interval", dict(type=int, default=None)),
        ("--critic-load", dict(type=str, default=None)), ("--critic-save", dict(type=str, default=None)),
        ("--save-hf", dict(type=str, default=None)), ("--save-hf-dtype", dict(type=str, default="bf16", choices=["bf16", "fp8"])),
        ("--save-hf-fp8-block-size", dict(type=int, default=128)), ("--save-hf-post-hook-path", dict(type=str, default=None)),
        ("--no-save-optim", _b()), ("--only-load-weight", _b()), ("--reset-optimizer-states", _b()),
        ("--async-save", _b()), ("--rotate-ckpt", _b()), ("--max-actor-ckpt-to-keep", dict(type=int, default=None)),
        ("--megatron-to-hf-mode", dict(type=str, default="raw", choices=["raw", "bridge"])),
    ],
    "rollout": [
        ("--prompt-data", dict(type=str, default=None)), ("--input-key", dict(type=str, default="input")),
        ("--label-key", dict(type=str, default=None)), ("--metadata-key", dict(type=str, default="metadata")),
        ("--attention-output-gate", _b()), ("--use-gated-attention", _b()), ("--apply-layernorm-1p", _b()), ("--rotary-percent", dict(type=float, default=None)),
        ("--tool-key", dict(type=str, default=None)), ("--apply-chat-template", _b()),
        ("--multimodal-keys", dict(type=json.loads, default=None)),      # {"image": "<row field with the image path(s)>"}
        ("--apply-chat-template-kwargs", dict(type=json.loads, default={})), ("--system-prompt", dict(type=str, default=None)),
        ("--rollout-batch-size", dict(type=int, default=None)), ("--n-samples-per-prompt", dict(type=int, default=1)),
        ("--over-sampling-batch-size", dict(type=int, default=None)),
        ("--rollout-max-prompt-len", dict(type=int, default=None)), ("--rollout-max-response-len", dict(type=int, default=1024)),
        ("--rollout-max-context-len", dict(type=int, default=None)),
        ("--rollout-temperature", dict(type=float, default=1.0)), ("--rollout-top-p", dict(type=float, default=1.0)),
        ("--rollout-top-k", dict(type=int, default=-1)), ("--rollout-stop", dict(type=str, nargs="*", default=None)),
        ("--rollout-stop-token-ids", dict(type=int, nargs="*", default=None)), ("--rollout-skip-special-tokens", _b()),
        ("--rollout-shuffle", _b()), ("--rollout-seed", dict(type=int, default=42)),
        ("--rollout-function-path", dict(type=str, default=None)),
        ("--custom-generate-function-path", dict(type=str, default=None)),
        ("--rollout-data-postprocess-path", dict(type=str, default=None)), ("--rollout-sample-filter-path", dict(type=str, default=None)),
        ("--dynamic-sampling-filter-path", dict(type=str, default=None)), ("--buffer-filter-path", dict(type=str, default=None)),
        ("--partial-rollout", _b()), ("--partial-rollout-max-aborted-count", dict(type=int, default=None)),
        ("--mask-offpolicy-in-partial-rollout", _b()),
        ("--rollout-external", _b()), ("--rollout-external-engine-addrs", dict(type=str, nargs="*", default=None)),
        ("--rollout-engine-init-timeout", dict(type=int, default=600)), ("--rollout-http-timeout", dict(type=float, default=None)),
        ("--use-rollout-routing-replay", _b()), ("--use-routing-replay", _b()), ("--use-rollout-logprobs", _b()),
        ("--use-rollout-entropy", _b()), ("--disable-rollout-global-dataset", _b()), ("--disable-rollout-trim-samples", _b()),
        ("--use-streaming-dataset", _b()), ("--streaming-buffer-size", dict(type=int, default=10000)),
        ("--use-agentic-rollout", _b()), ("--agentic-concurrency", dict(type=int, default=None)),
        # agents as external commands (relax/utils/arguments.py:1421-1552)
        ("--agent-command", dict(type=str, default=None)), ("--agent-cwd", dict(type=str, default=None)),
        ("--agent-timeout", dict(type=float, default=1800.0)), ("--agent-env", dict(type=str, nargs="+", default=[])),
        ("--agentic-program-admission", _b()), ("--agentic-admission-headroom", dict(type=float, default=0.90)),
        ("--agentic-admission-expected-decode-cap", dict(type=int, default=None)),
        ("--agentic-admission-pressure-threshold", dict(type=float, default=0.92)),
        ("--agentic-admission-max-wait-s", dict(type=float, default=30.0)),
        ("--agentic-admission-scope", dict(type=str, default="train", choices=["train", "all"])),
        ("--agentic-eval-concurrency", dict(type=int, default=None)), ("--agentic-prelaunch", _b()),
        ("--agentic-session-lifecycle", _b()), ("--agentic-tool-call-parser", dict(type=str, default=None)),
        ("--agentic-reasoning-parser", dict(type=str, default=None)), ("--agentic-custom-advantage-path", dict(type=str, default=None)),
    ],
    "fault_tolerance": [
        ("--use-fault-tolerance", _b()), ("--use-health-check", _b()), ("--max-global-restart", dict(type=int, default=3)),
        ("--rollout-health-check-interval", dict(type=float, default=30.0)), ("--rollout-health-check-timeout", dict(type=float, default=30.0)),
        ("--rollout-health-check-first-wait", dict(type=float, default=0.0)),
        ("--rollout-health-check-max-consecutive-failures", dict(type=int, default=3)),
        ("--scale-out-timeout", dict(type=float, default=1800.0)), ("--scale-in-drain-timeout", dict(type=float, default=300.0)),
        ("--scale-in-shutdown-timeout", dict(type=float, default=60.0)), ("--scale-weight-sync-precheck", _b()),
        ("--scale-out-partial-success-policy", dict(type=str, default="keep", choices=["keep", "rollback"])),
        ("--autoscaler-config", dict(type=str, default=None)),
        # external engines only: the control endpoints of the elastic pool (/scale_out, /scale_in, /engines) and further
        # pre-launched servers the autoscaler may bring in
        ("--elastic-control-port", dict(type=int, default=None)), ("--rollout-standby-engine-addrs", dict(type=str, nargs="*", default=None)),
        ("--autoscaler-interval", dict(type=float, default=15.0)),
    ],
    "eval": [
        ("--eval-interval", dict(type=int, default=None)), ("--eval-prompt-data", dict(type=str, nargs="*", default=None)),
        ("--eval-config", dict(type=str, default=None)), ("--skip-eval-before-train", _b()),
        ("--n-samples-per-eval-prompt", dict(type=int, default=1)), ("--eval-temperature", dict(type=float, default=None)),
        ("--eval-top-p", dict(type=float, default=None)), ("--eval-top-k", dict(type=int, default=None)),
        ("--eval-max-response-len", dict(type=int, default=None)), ("--eval-max-prompt-len", dict(type=int, default=None)),
        ("--eval-input-key", dict(type=str, default=None)), ("--eval-label-key", dict(type=str, default=None)),
        ("--eval-reward-key", dict(type=str, default=None)), ("--eval-size", dict(type=int, default=None)),
        ("--log-passrate", _b()),
    ],
    "algo": [
        ("--advantage-estimator", dict(type=str, default="grpo", choices=ADVANTAGE_ESTIMATORS)),
        ("--loss-type", dict(type=str, default="policy_loss", choices=LOSS_TYPES)),
        ("--custom-loss-function-path", dict(type=str, default=None)),
        ("--eps-clip", dict(type=float, default=0.2)), ("--eps-clip-high", dict(type=float, default=None)),
        ("--eps-clip-c", dict(type=float, default=None)), ("--value-clip", dict(type=float, default=0.2)),
        ("--kl-coef", dict(type=float, default=0.0)), ("--use-kl-loss", _b()), ("--kl-loss-coef", dict(type=float, default=0.0)),
        ("--kl-loss-type", dict(type=str, default="k1", choices=["k1", "k2", "k3", "low_var_kl"])), ("--use-unbiased-kl", _b()),
        ("--entropy-coef", dict(type=float, default=0.0)), ("--gamma", dict(type=float, default=1.0)), ("--lambd", dict(type=float, default=1.0)),
        ("--normalize-advantages", _b()), ("--disable-grpo-std-normalization", _b()), ("--disable-rewards-normalization", _b()),
        ("--disable-compute-advantages-and-returns", _b()),
        ("--use-tis", _b()), ("--tis-clip", dict(type=float, default=2.0)), ("--tis-clip-low", dict(type=float, default=0.0)),
        ("--custom-tis-function-path", dict(type=str, default=None)), ("--custom-pg-loss-reducer-function-path", dict(type=str, default=None)),
        ("--get-mismatch-metrics", _b()), ("--use-opsm", _b()), ("--opsm-delta", dict(type=float, default=1e-4)),
        ("--sapo-tau-pos", dict(type=float, default=1.0)), ("--sapo-tau-neg", dict(type=float, default=1.05)),
        ("--m2po-kl2-budget", dict(type=float, default=0.04)), ("--m2po-miniclip-low", dict(type=float, default=0.3)),
        ("--m2po-miniclip-high", dict(type=float, default=0.5)),
        ("--num-critic-only-steps", dict(type=int, default=0)), ("--critic-lr", dict(type=float, default=None)),
        ("--critic-lr-warmup-iters", dict(type=int, default=0)), ("--critic-train-only", _b()),
        ("--optimize-routing-replay", _b()),
    ],
    "reward": [
        ("--rm-type", dict(type=str, default=None)), ("--rm-url", dict(type=str, default=None)),
        ("--custom-rm-path", dict(type=str, default=None)), ("--group-rm", _b()), ("--reward-key", dict(type=str, default=None)),
        ("--custom-reward-post-process-path", dict(type=str, default=None)), ("--reward-num-workers", dict(type=int, default=8)),
        ("--reward-max-concurrency", dict(type=int, default=64)), ("--defer-reward-to-post-process", _b()),
        ("--genrm-model-path", dict(type=str, default=None)), ("--genrm-num-gpus", dict(type=int, default=0)),
        ("--genrm-num-gpus-per-engine", dict(type=int, default=1)),
        ("--genrm-engine-addrs", dict(type=str, nargs="*", default=None)),     # grader engine servers on their own GPUs
    ],
    "opd": [
        ("--opd-type", dict(type=str, default=None, choices=[None, "sglang", "megatron", "opsd"])),
        ("--opd-kl-coef", dict(type=float, default=1.0)), ("--opd-teacher-load", dict(type=str, default=None)),
        ("--opd-teacher-urls", dict(type=str, nargs="*", default=None)), ("--opd-topk", dict(type=int, default=0)),
        # relax/utils/opd/opd_utils.py add_opd_arguments :466-680
        ("--use-opd", _b()), ("--opd-teacher-url", dict(type=str, default=None)),
        ("--opd-token-selection", dict(type=str, default="student_sampled", choices=["student_sampled", "student_topk", "teacher_topk", "union"])),
        ("--opd-log-prob-top-k", dict(type=int, default=0)),
        ("--opd-kl-type", dict(type=str, default="reverse_kl", choices=["reverse_kl", "forward_kl", "jsd", "low_var_kl"])),
        ("--opd-jsd-alpha", dict(type=float, default=0.5)), ("--opd-norm-mode", dict(type=str, default="tail", choices=["tail", "norm", "trunc"])),
        ("--opd-log-prob-min-clamp", dict(type=float, default=None)), ("--opd-per-token-clip", dict(type=float, default=None)),
        ("--opd-loss-coef", dict(type=float, default=0.0)), ("--opd-only-reward", _b()), ("--opd-is-clip", dict(type=float, default=None)),
    ],
    "lora": [
        ("--lora-rank", dict(type=int, default=0)), ("--lora-alpha", dict(type=float, default=16.0)),
        ("--lora-dropout", dict(type=float, default=0.0)), ("--lora-target-modules", dict(type=str, nargs="*", default=None)),
        ("--lora-adapter-mode", _b()), ("--lora-merge-mode", _b()),
    ],
    "router": [
        ("--use-slime-router", _b()), ("--slime-router-sticky", _b()), ("--slime-router-timeout", dict(type=float, default=None)),
        ("--slime-router-max-connections", dict(type=int, default=None)),
        ("--slime-router-health-check-failure-threshold", dict(type=int, default=3)),
        ("--slime-router-middleware-paths", dict(type=str, nargs="*", default=None)),
    ],
    "logging": [
        ("--use-wandb", _b()), ("--wandb-project", dict(type=str, default=None)), ("--wandb-group", dict(type=str, default=None)),
        ("--use-tensorboard", _b()), ("--tb-project-name", dict(type=str, default=None)), ("--tb-experiment-name", dict(type=str, default=None)),
        ("--use-clearml", _b()), ("--notify-urls", dict(type=str, nargs="*", default=None)),
        ("--use-metrics-service", _b()), ("--timeline-dump-dir", dict(type=str, default=None)),
        ("--log-multi-turn", _b()), ("--log-reward-category", dict(type=str, default=None)),
        ("--profile-target", dict(type=str, nargs="*", default=None)), ("--profile-step-start", dict(type=int, default=None)),
        ("--profile-step-end", dict(type=int, default=None)), ("--profile-with-stack", _b()), ("--profile-with-memory", _b()),
        ("--profile-with-flops", _b()), ("--record-memory-history", _b()), ("--memory-snapshot-dir", dict(type=str, default=None)),
        ("--memory-snapshot-num-steps", dict(type=int, default=None)),
    ],
    "ci": [
        ("--ci-test", _b()), ("--ci-save-grad-norm", dict(type=str, default=None)), ("--ci-load-grad-norm", dict(type=str, default=None)),
        ("--ci-disable-kl-checker", _b()),
    ],
    "mtp": [
        ("--enable-mtp-training", _b()), ("--mtp-num-layers", dict(type=int, default=None)),
        ("--mtp-loss-scaling-factor", dict(type=float, default=0.1)), ("--mtp-only-training", _b()),
    ],
    "sft": [
        ("--sft-predict-interval", dict(type=int, default=None)),
        ("--sft-chunked-logits", _b()), ("--sft-logits-chunk-size", dict(type=int, default=4096)),
        ("--sft-max-in-flight-steps", dict(type=int, default=2)), ("--sft-prefetch-buffer-size", dict(type=int, default=64)),
        ("--loss-mask-type", dict(type=str, default="qwen")), ("--num-labels", dict(type=int, default=None)),
        ("--problem-type", dict(type=str, default=None)), ("--classification-threshold", dict(type=float, default=0.5)),
    ],
    # Megatron-named model / parallel / optimizer flags
    "model": [
        ("--model-name", dict(type=str, default=None)), ("--num-layers", dict(type=int, default=None)),
        ("--hidden-size", dict(type=int, default=None)), ("--ffn-hidden-size", dict(type=int, default=None)),
        ("--num-attention-heads", dict(type=int, default=None)), ("--num-query-groups", dict(type=int, default=None)),
        ("--kv-channels", dict(type=int, default=None)), ("--vocab-size", dict(type=int, default=None)),
        ("--padded-vocab-size", dict(type=int, default=None)), ("--norm-epsilon", dict(type=float, default=None)),
        ("--rotary-base", dict(type=float, default=None)), ("--qk-layernorm", _b()), ("--add-qkv-bias", _b()),
        ("--swiglu", _b(True)), ("--group-query-attention", _b(True)), ("--untie-embeddings-and-output-weights", _b()),
        ("--num-experts", dict(type=int, default=None)), ("--moe-router-topk", dict(type=int, default=None)),
        ("--moe-ffn-hidden-size", dict(type=int, default=None)), ("--moe-aux-loss-coeff", dict(type=float, default=None)),
        ("--moe-token-dispatcher-type", dict(type=str, default="alltoall")), ("--moe-grouped-gemm", _b()),
        ("--moe-permute-fusion", _b()), ("--attention-backend", dict(type=str, default="flash")),
        ("--bf16", _b(True)), ("--fp16", _b()), ("--fp8-format", dict(type=str, default=None)), ("--fp8-recipe", dict(type=str, default=None)),
    ],
    "parallel": [
        ("--tensor-model-parallel-size", dict(type=int, default=1)), ("--pipeline-model-parallel-size", dict(type=int, default=1)),
        ("--context-parallel-size", dict(type=int, default=1)), ("--expert-model-parallel-size", dict(type=int, default=1)),
        ("--expert-tensor-parallel-size", dict(type=int, default=None)), ("--sequence-parallel", _b()),
        ("--use-distributed-optimizer", _b(True)), ("--overlap-grad-reduce", _b()), ("--overlap-param-gather", _b()),
        ("--recompute-granularity", dict(type=str, default=None, choices=[None, "full", "selective"])),
        ("--recompute-method", dict(type=str, default=None)), ("--recompute-num-layers", dict(type=int, default=None)),
        ("--dynamic-context-parallel", _b()), ("--optimizer-cpu-offload", _b()),
        ("--accumulate-allreduce-grads-in-fp32", _b(True)),
    ],
    "optimizer": [
        ("--lr", dict(type=float, default=1e-6)), ("--min-lr", dict(type=float, default=0.0)),
        ("--lr-decay-style", dict(type=str, default="constant", choices=["constant", "linear", "cosine"])),
        ("--lr-warmup-iters", dict(type=int, default=0)), ("--lr-decay-iters", dict(type=int, default=None)),
        ("--weight-decay", dict(type=float, default=0.01)), ("--adam-beta1", dict(type=float, default=0.9)),
        ("--adam-beta2", dict(type=float, default=0.999)), ("--adam-eps", dict(type=float, default=1e-8)),
        ("--clip-grad", dict(type=float, default=1.0)), ("--store-param-remainders", _b(True)),
        ("--no-store-param-remainders", dict(action="store_false", dest="store_param_remainders")),
    ],
}

# rollout-engine flags accepted under the reference's prefix (backends/sglang/arguments.py) -> engine option
ENGINE_FLAGS = {
    "--sglang-mem-fraction-static": ("engine_mem_fraction", float, 0.8),
    "--sglang-context-length": ("engine_context_length", int, None),
    "--sglang-server-concurrency": ("engine_concurrency", int, 512),
    "--sglang-max-running-requests": ("engine_max_running", int, 256),
    "--sglang-chunked-prefill-size": ("engine_max_prefill_tokens", int, 16384),
    "--sglang-page-size": ("engine_block_size", int, 16),
    "--sglang-disable-cuda-graph": ("engine_disable_cuda_graph", "flag", False),
    "--sglang-disable-radix-cache": ("engine_disable_prefix_sharing", "flag", False),
    "--sglang-enable-memory-saver": ("engine_memory_saver", "flag", False),
    "--sglang-tp-size": ("engine_tp", int, None), "--sglang-ep-size": ("engine_ep", int, 1),
    "--sglang-dp-size": ("engine_dp", int, 1), "--sglang-pp-size": ("engine_pp", int, 1),
    "--sglang-enable-return-routed-experts": ("engine_return_routed_experts", "flag", False),
    # speculative decoding drafted by the model's MTP block (rollout/speculative.py): num-steps chained proposals per pass
    "--sglang-speculative-algorithm": ("engine_speculative_algorithm", str, None),
    "--sglang-speculative-num-steps": ("engine_speculative_num_steps", int, 1),
    "--sglang-speculative-eagle-topk": ("engine_speculative_eagle_topk", int, 1),
    "--sglang-speculative-num-draft-tokens": ("engine_speculative_num_draft_tokens", int, 2),
}


# ---------------------------------------------------------------------------------------------------------------
# Flags of the reference's recipes that this build accepts but does not (fully) implement.  A recipe must never
# run with different math, precision or layout than it asks for without saying so:
#   "raise": the flag changes what is computed or where; a non-default value stops the run at parse time.
#   "warn":  the flag tunes an operational detail (a timeout, a concurrency cap, a library choice) that has no
#            counterpart here or is always on; a non-default value is reported once and the run goes on.
# Everything not listed is consumed by the controller, the trainer, the rollout engine or a service.
_R, _W = "raise", "warn"
FLAG_POLICY: dict[str, tuple] = {
    # numerics / layout
    "--fp8-format": (_R, "fp8 training is not wired (the block-scaled fp8 GEMM exists as an operator only)"),
    "--fp8-recipe": (_R, "fp8 training is not wired"),
    "--optimizer-cpu-offload": (_R, "optimizer state lives on the GPU (or is offloaded whole between phases with --offload-train)"),
    "--expert-tensor-parallel-size": (_R, "experts are not tensor-parallel here (expert TP = 1)"),
    "--qkv-format": (_R, "only the packed thd layout is implemented"),
    "--padded-vocab-size": (_R, "the vocabulary is padded to a multiple of the tensor-parallel size only"),
    "--train-backend": (_R, "there is one trainer (this package); Megatron-LM is not used"),
    # rollout behaviour
    "--sglang-dp-size": (_R, "rollout engines are replicated per engine group, not data-parallel inside one engine"),
    # algorithm
    "--genrm-num-gpus": (_R, "grader engines either share the rollout ranks (--genrm-model-path) or run as engine servers on their own "
                             "GPUs, started with `serve engine` and named by --genrm-engine-addrs; this job does not launch them"),
    # operational, no effect here
    "--async-save": (_W, "checkpoints are written synchronously"),
    "--attention-backend": (_W, "there is one attention implementation (tcgen05 flash attention)"),
    "--moe-grouped-gemm": (_W, "always on"), "--moe-permute-fusion": (_W, "always on"),
    "--moe-token-dispatcher-type": (_W, "all-to-all dispatch is the only dispatcher"),
    "--overlap-grad-reduce": (_W, "the gradient reduce-scatter is fused into the optimizer kernel"),
    "--overlap-param-gather": (_W, "the parameter all-gather is fused into the optimizer kernel"),
    "--recompute-method": (_W, "--recompute-granularity full recomputes every layer"),
    "--recompute-num-layers": (_W, "--recompute-granularity full recomputes every layer"),
    "--log-probs-chunk-size": (_W, "the fused LM head never materialises the logits"),
    "--sglang-speculative-num-draft-tokens": (_W, "a verify pass carries --sglang-speculative-num-steps + 1 rows per request (one chain of proposals)"),
    "--sglang-server-concurrency": (_W, None), "--agentic-prelaunch": (_W, "agents start when their sample is scheduled"),
    "--agentic-session-lifecycle": (_W, "a session's cache entries are released by the engine's own eviction"),
    "--agentic-eval-concurrency": (_W, None), "--agentic-admission-expected-decode-cap": (_W, None),
    "--agentic-admission-scope": (_W, None),
    "--sglang-mem-fraction-static": (_W, "the KV cache is sized from the batch shape"),
    "--critic-num-nodes": (_W, "the critic shares the actor's ranks"),
    "--critic-num-gpus-per-node": (_W, "the critic shares the actor's ranks"),
    "--disable-rollout-trim-samples": (_W, None), "--disable-weights-backuper": (_W, None),
    "--enable-affinity": (_W, "no Ray node affinity"), "--genrm-num-gpus-per-engine": (_W, None),
    "--log-multi-turn": (_W, None), "--log-reward-category": (_W, None), "--loss-mask-type": (_W, None),
    "--megatron-to-hf-mode": (_W, "one converter"), "--optimize-routing-replay": (_W, None),
    "--profile-target": (_W, "the trainer is the profiled role"), "--reward-max-concurrency": (_W, None),
    "--reward-num-workers": (_W, None), "--rollout-engine-init-timeout": (_W, None), "--rollout-http-timeout": (_W, None),
    "--rollout-skip-special-tokens": (_W, None), "--selective-offload": (_W, None), "--sft-chunked-logits": (_W, "always on"),
    "--sft-logits-chunk-size": (_W, None), "--sft-max-in-flight-steps": (_W, None),
    "--slime-router-health-check-failure-threshold": (_W, None), "--slime-router-max-connections": (_W, None),
    "--slime-router-middleware-paths": (_W, None), "--slime-router-sticky": (_W, None), "--slime-router-timeout": (_W, None),
    "--use-slime-router": (_W, "the in-process router is used when several engines serve one rank; the HTTP proxy is `serve router`"),
    "--train-env-vars": (_W, None), "--train-memory-margin-bytes": (_W, None), "--update-weight-buffer-size": (_W, None),
    "--scale-in-shutdown-timeout": (_W, "external engines are drained and forgotten, not shut down"),
}
_WARNED: set = set()


def apply_flag_policy(a: argparse.Namespace, parser: Optional[argparse.ArgumentParser] = None, warn=None) -> list:
    """Stop on (or report) accepted-but-unimplemented flags that were given a non-default value.
    Returns the warnings issued (for tests)."""
    import warnings as _warnings

    parser = parser or build_parser()
    by_flag = {}
    for act in parser._actions:
        for opt in act.option_strings:
            by_flag[opt] = act
    out = []
    for flag, (kind, why) in FLAG_POLICY.items():
        act = by_flag.get(flag)
        if act is None:
            continue
        val = getattr(a, act.dest, act.default)
        if val == act.default or (val in (None, [], {}, 0, False) and act.default in (None, [], {}, 0, False)):
            continue
        if flag in ("--expert-tensor-parallel-size",) and val in (None, 1):
            continue
        if flag == "--sglang-dp-size" and val in (None, 1):
            continue
        if flag == "--sglang-speculative-num-draft-tokens" and val == (getattr(a, "engine_speculative_num_steps", 1) or 1) + 1:
            continue            # exactly what one chain of that many proposals needs
        if flag == "--genrm-num-gpus" and getattr(a, "genrm_engine_addrs", None):
            continue            # the GPUs are the ones behind the named servers
        msg = f"{flag}={val!r} is accepted for recipe compatibility but not implemented here" + (f": {why}" if why else "")
        if kind == _R:
            raise ValueError(msg)
        if flag not in _WARNED:
            _WARNED.add(flag)
            (warn or _warnings.warn)(msg)
        out.append(msg)
    return out


def _freeze_list(a) -> Optional[list]:
    """``--freeze-params-name-list`` plus the three multimodal switches (relax/utils/arguments.py:443-455) as name
    patterns: the vision tower lives under ``vision.``, its projection into the language model is the merger."""
    out = list(getattr(a, "freeze_params_name_list", None) or [])
    if getattr(a, "freeze_language_model", False):
        out.append(r"^(?!vision\.)")
    if getattr(a, "freeze_vision_model", False):
        out.append(r"^vision\.(?!merger_)")
    if getattr(a, "freeze_vision_projection", False):
        out.append(r"^vision\.merger_")
    return out or None


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("relax_b200", allow_abbrev=False)
    for group, flags in FLAGS.items():
        g = p.add_argument_group(group)
        for name, kw in flags:
            g.add_argument(name, **kw)
    g = p.add_argument_group("rollout engine")
    for name, (dest, typ, default) in ENGINE_FLAGS.items():
        if typ == "flag":
            g.add_argument(name, dest=dest, action="store_true", default=default)
        else:
            g.add_argument(name, dest=dest, type=typ, default=default)
    return p


def parse_resource(spec: Optional[str]) -> dict:
    """``--resource`` JSON -> {role: (num_serves, num_gpus)}."""
    if not spec:
        return {}
    d = json.loads(spec) if isinstance(spec, str) else dict(spec)
    out = {}
    for role, v in d.items():
        if not (isinstance(v, (list, tuple)) and len(v) == 2):
            raise ValueError(f"--resource entry for {role!r} must be [num_serves, num_gpus], got {v!r}")
        out[role] = (int(v[0]), int(v[1]))
    return out


def validate_args(a: argparse.Namespace) -> argparse.Namespace:
    """Mode rules and derived values (relax/utils/arguments.py:3230-3971)."""
    # --- modes
    if a.hybrid:
        a.fully_async, a.colocate = True, True            # hybrid = separate pools, in-process ref/actor_fwd
    elif a.fully_async and a.colocate:
        raise ValueError("--fully-async and --colocate are mutually exclusive (use --hybrid for in-process forward roles)")
    if a.colocate and not a.fully_async and a.max_staleness != 0:
        raise ValueError("colocated (synchronous) training requires --max-staleness 0")
    if a.offload:
        a.offload_train = a.offload_rollout = True
    if a.offload_train is None:
        a.offload_train = bool(a.colocate and not a.hybrid)
    if a.offload_rollout is None:
        a.offload_rollout = bool(a.colocate and not a.hybrid)
    # --- resources
    a.resource_map = parse_resource(a.resource)
    if a.resource_map:
        if "actor" in a.resource_map:
            gpus = a.resource_map["actor"][1]
            a.actor_num_nodes = max(1, gpus // a.num_gpus_per_node)
            a.actor_num_gpus_per_node = min(gpus, a.num_gpus_per_node)
        if "rollout" in a.resource_map and a.rollout_num_gpus is None:
            a.rollout_num_gpus = a.resource_map["rollout"][1]
        if a.colocate and not a.hybrid and "actor" in a.resource_map and "rollout" in a.resource_map:
            if a.resource_map["actor"][1] != a.resource_map["rollout"][1]:
                raise ValueError("colocated actor and rollout must be given the same GPUs")
    if a.rollout_num_gpus is None:
        a.rollout_num_gpus = a.actor_num_nodes * a.actor_num_gpus_per_node
    if a.rollout_num_gpus % a.rollout_num_gpus_per_engine:
        raise ValueError("--rollout-num-gpus must be a multiple of --rollout-num-gpus-per-engine")
    if a.engine_tp is None:
        a.engine_tp = a.rollout_num_gpus_per_engine // max(1, a.engine_pp)
    # --- algorithm
    if a.eps_clip_high is None:
        a.eps_clip_high = a.eps_clip
    if a.eps_clip_c is not None and a.eps_clip_c <= 1.0:
        raise ValueError("--eps-clip-c (dual clip) must be > 1")
    if a.advantage_estimator == "rloo" and a.n_samples_per_prompt < 2:
        raise ValueError("RLOO needs --n-samples-per-prompt >= 2")
    if a.advantage_estimator in ("gspo",) and a.calculate_per_token_loss:
        raise ValueError("GSPO uses sequence-level ratios; --calculate-per-token-loss is not supported with it")
    if a.use_kl_loss and a.kl_coef != 0:
        raise ValueError("choose either the KL loss term (--use-kl-loss) or reward shaping (--kl-coef), not both")
    if a.use_tis and a.true_on_policy_mode:
        raise ValueError("--use-tis needs old-policy log-probs, which --true-on-policy-mode skips")
    a.rewards_normalization = not a.disable_rewards_normalization
    a.grpo_std_normalization = not a.disable_grpo_std_normalization
    if a.loss_type == "custom_loss" and not a.custom_loss_function_path:
        raise ValueError("--loss-type custom_loss needs --custom-loss-function-path")
    if a.advantage_estimator == "ppo" and a.resource_map and "critic" not in a.resource_map:
        raise ValueError("PPO needs a critic entry in --resource")
    # --- batch arithmetic
    if a.rollout_batch_size is not None:
        per_rollout = a.rollout_batch_size * a.n_samples_per_prompt
        if a.global_batch_size is None:
            steps = a.num_steps_per_rollout or 1
            if per_rollout % steps:
                raise ValueError("rollout_batch_size * n_samples_per_prompt must divide by num_steps_per_rollout")
            a.global_batch_size = per_rollout // steps
        elif a.num_steps_per_rollout is None and not a.use_dynamic_global_batch_size:
            if per_rollout % a.global_batch_size:
                raise ValueError(f"samples per rollout ({per_rollout}) must be a multiple of --global-batch-size ({a.global_batch_size})")
            a.num_steps_per_rollout = per_rollout // a.global_batch_size
    # --- on-policy distillation
    if a.use_opd and not a.opd_type:
        a.opd_type = "sglang" if (a.opd_teacher_urls or a.opd_teacher_url) else "megatron"
    if a.opd_teacher_url and not a.opd_teacher_urls:
        a.opd_teacher_urls = [a.opd_teacher_url]
    if a.opd_topk and not a.opd_log_prob_top_k:          # short form: the teacher's top-K ids
        a.opd_log_prob_top_k = a.opd_topk
        if a.opd_token_selection == "student_sampled":
            a.opd_token_selection = "teacher_topk"
    if not a.opd_type:
        a.opd_loss_coef = 0.0
    if a.opd_type and (a.opd_loss_coef or 0.0) != 0.0:
        # relax/utils/opd/opd_utils.py:719-731: the signal enters through the advantages OR as a loss term
        if a.opd_kl_coef not in (0.0, 1.0):          # 1.0 is the flag's default: loss mode overrides it
            raise ValueError("exactly one of --opd-kl-coef / --opd-loss-coef is non-zero (advantage mode or loss mode)")
        a.opd_kl_coef = 0.0
        if a.opd_token_selection != "student_sampled":
            raise ValueError("--opd-loss-coef (loss mode) is wired for the sampled token; top-K selections use --opd-kl-coef")
    for name in ("opd_per_token_clip", "opd_is_clip"):
        if getattr(a, name) is not None and getattr(a, name) <= 0:
            raise ValueError(f"--{name.replace('_', '-')} must be > 0")
    if a.opd_token_selection != "student_sampled":
        if a.opd_log_prob_top_k <= 0:
            raise ValueError(f"--opd-token-selection {a.opd_token_selection} needs --opd-log-prob-top-k > 0")
        if a.opd_teacher_urls:
            raise ValueError("top-K token selections need an in-process teacher (--opd-teacher-load): remote teachers return "
                             "the sampled token's log-prob only")
        if a.opd_kl_type == "low_var_kl" and a.opd_token_selection == "union":
            pass
    elif a.opd_kl_type in ("forward_kl", "jsd"):
        raise ValueError(f"--opd-kl-type {a.opd_kl_type} needs both distributions: choose a top-K --opd-token-selection")
    if a.engine_speculative_algorithm:
        if a.engine_speculative_algorithm.upper() not in ("EAGLE", "NEXTN", "MTP"):
            raise ValueError("--sglang-speculative-algorithm: the draft model is the policy's own MTP block (EAGLE / NEXTN)")
        if not (a.mtp_num_layers or 0) and not a.hf_checkpoint:
            raise ValueError("speculative decoding drafts with the multi-token-prediction block: set --mtp-num-layers")
        if a.engine_speculative_eagle_topk != 1:
            raise ValueError("--sglang-speculative-eagle-topk: one chain of proposals (top-k 1) is implemented")
    if a.rollout_external:
        if not a.rollout_external_engine_addrs:
            raise ValueError("--rollout-external needs --rollout-external-engine-addrs host:port [host:port ...]")
        if getattr(a, "fully_async", False) and not getattr(a, "hybrid", False):
            raise ValueError("--rollout-external drives pre-launched engines from the colocated loop (--colocate)")
    elif a.rollout_external_engine_addrs:
        raise ValueError("--rollout-external-engine-addrs has no effect without --rollout-external")
    if (a.autoscaler_config or a.elastic_control_port is not None or a.rollout_standby_engine_addrs) and not a.rollout_external:
        raise ValueError("--autoscaler-config / --elastic-control-port / --rollout-standby-engine-addrs scale a pool of "
                         "pre-launched engine servers: add --rollout-external --rollout-external-engine-addrs ...")
    if a.use_agentic_rollout:
        # relax/utils/arguments.py:3015-3017 points the rollout function at the agentic entry; same here
        if not a.agent_command or not a.agent_cwd:
            raise ValueError("--use-agentic-rollout needs --agent-command and --agent-cwd")
        if a.custom_generate_function_path:
            raise ValueError("--use-agentic-rollout installs its own generate function; drop --custom-generate-function-path")
        a.custom_generate_function_path = "relax_b200.rollout.agent_pipeline:command_generate"
        from ..rollout.openai_api import parse_tool_calls, split_reasoning

        if a.agentic_tool_call_parser:
            parse_tool_calls("", a.agentic_tool_call_parser)         # unknown names stop here, not in the first rollout
        if a.agentic_reasoning_parser:
            split_reasoning("", a.agentic_reasoning_parser)
        if a.agentic_concurrency is None:
            a.agentic_concurrency = getattr(a, "over_sampling_batch_size", None) or a.rollout_batch_size or 32
    if (a.num_iters_per_train_update or 1) > 1:
        # relax/utils/arguments.py:246-250: "fully async pipeline num of iters every global batch"
        if not (getattr(a, "fully_async", False) or getattr(a, "hybrid", False)):
            raise ValueError("--num-iters-per-train-update > 1 streams parts of a rollout batch to the trainer: it needs --fully-async")
        if a.rollout_batch_size is not None and a.rollout_batch_size % a.num_iters_per_train_update:
            raise ValueError("--rollout-batch-size must divide by --num-iters-per-train-update (whole prompt groups per part)")
    if a.use_dynamic_batch_size and a.max_tokens_per_gpu is None:
        raise ValueError("--use-dynamic-batch-size needs --max-tokens-per-gpu")
    if a.log_probs_max_tokens_per_gpu is None:
        a.log_probs_max_tokens_per_gpu = a.max_tokens_per_gpu
    # --- parallel
    if a.tensor_model_parallel_size > 1:
        a.sequence_parallel = True
    if a.dynamic_context_parallel and a.context_parallel_size < 2:
        raise ValueError("--dynamic-context-parallel needs --context-parallel-size >= 2")
    if a.fp16:
        a.bf16 = False
    # --- LR schedule length (relax/backends/megatron/model.py:220-265)
    if a.num_rollout and a.rollout_batch_size and a.global_batch_size:
        a.train_iters = a.num_rollout * a.rollout_batch_size * a.n_samples_per_prompt // a.global_batch_size
        if a.lr_decay_iters is None:
            a.lr_decay_iters = a.train_iters
    if getattr(a, "dump_details", None):       # one switch for both debug dumps (relax/utils/arguments.py:3542-3544)
        a.save_debug_rollout_data = a.save_debug_rollout_data or f"{a.dump_details}/rollout_data"
        a.save_debug_train_data = a.save_debug_train_data or f"{a.dump_details}/train_data"
    if a.partial_rollout and not a.over_sampling_batch_size:
        a.over_sampling_batch_size = a.rollout_batch_size
    if a.rm_type is None and a.custom_rm_path is None and not a.debug_train_only:
        a.rm_type = "parity"
    return a


def parse_args(argv: Optional[Sequence[str]] = None) -> argparse.Namespace:
    parser = build_parser()
    a = parser.parse_args(argv)
    apply_flag_policy(a, parser)
    return validate_args(a)


def model_config_from_args(a):
    """Model preset by ``--model-name`` with explicit shape flags overriding it."""
    from ..models.config import ModelConfig, get_config

    over = {}
    m = [("num_layers", "num_layers"), ("hidden_size", "hidden_size"), ("ffn_hidden_size", "ffn_hidden_size"),
         ("num_attention_heads", "num_attention_heads"), ("num_query_groups", "num_query_groups"),
         ("kv_channels", "head_dim"), ("vocab_size", "vocab_size"), ("num_experts", "num_experts"),
         ("moe_router_topk", "moe_top_k"), ("moe_ffn_hidden_size", "moe_ffn_hidden_size"),
         ("mtp_num_layers", "mtp_num_layers")]
    for src, dst in m:
        v = getattr(a, src, None)
        if v is not None:
            over[dst] = v
    # Megatron-style shape switches of the reference's scripts/models/*.sh
    for src, dst in (("norm_epsilon", "rms_norm_eps"), ("rotary_base", "rope_theta"), ("moe_aux_loss_coeff", "moe_aux_loss_coef")):
        v = getattr(a, src, None)
        if v is not None:
            over[dst] = float(v)
    if a.model_name:          # a preset: the switches only add to it
        if getattr(a, "add_qkv_bias", False):
            over["qkv_bias"] = True
        if getattr(a, "qk_layernorm", False):
            over["qk_layernorm"] = True
        if getattr(a, "untie_embeddings_and_output_weights", False):
            over["tie_word_embeddings"] = False
    else:                     # a model given by shape flags alone: Megatron's meaning of the switches
        over["qkv_bias"] = bool(getattr(a, "add_qkv_bias", False))
        over["qk_layernorm"] = bool(getattr(a, "qk_layernorm", False))
        over["tie_word_embeddings"] = not getattr(a, "untie_embeddings_and_output_weights", False)
    if getattr(a, "attention_output_gate", False) or getattr(a, "use_gated_attention", False):
        over["attention_output_gate"] = True
    if getattr(a, "apply_layernorm_1p", False):
        over["layernorm_zero_centered"] = True
    if getattr(a, "rotary_percent", None) is not None:
        over["rotary_percent"] = float(a.rotary_percent)
    if getattr(a, "num_labels", None):
        over["num_classes"] = int(a.num_labels)       # sequence-classification head on the last token
    if a.model_name:
        return get_config(a.model_name, **over)
    return ModelConfig(name="custom", **over)


def _ci_config(a):
    from ..train.ci_utils import CIConfig

    ci = CIConfig.from_args(a)
    return ci if (ci.enabled or ci.save_grad_norm or ci.load_grad_norm) else None


def train_config_from_args(a):
    from ..algo.loss import LossConfig
    from ..train.actor import TrainConfig
    from ..train.optimizer import OptimizerConfig

    loss = LossConfig.from_args(a)
    optim = OptimizerConfig(lr=a.lr, min_lr=a.min_lr, weight_decay=a.weight_decay, adam_beta1=a.adam_beta1,
                            adam_beta2=a.adam_beta2, adam_eps=a.adam_eps, clip_grad=a.clip_grad,
                            lr_decay_style=a.lr_decay_style, lr_warmup_iters=a.lr_warmup_iters,
                            lr_decay_iters=a.lr_decay_iters,
                            grad_dtype="fp32" if a.accumulate_allreduce_grads_in_fp32 else "param",
                            split_master=a.store_param_remainders)
    return TrainConfig(
        advantage_estimator=a.advantage_estimator, global_batch_size=a.global_batch_size or 1,
        max_tokens_per_gpu=a.max_tokens_per_gpu or 8192, use_dynamic_batch_size=a.use_dynamic_batch_size,
        micro_batch_size=a.micro_batch_size, rollout_temperature=a.rollout_temperature,
        n_samples_per_prompt=a.n_samples_per_prompt, kl_coef=a.kl_coef, gamma=a.gamma, lambd=a.lambd,
        normalize_advantages=a.normalize_advantages, rewards_normalization=a.rewards_normalization,
        grpo_std_normalization=a.grpo_std_normalization, balance_data=a.balance_data,
        recompute=a.recompute_granularity == "full", pad_multiple=a.data_pad_size_multiplier,
        use_rollout_logprobs=a.use_rollout_logprobs, keep_old_actor=a.keep_old_actor,
        enable_mtp_training=a.enable_mtp_training, mtp_loss_scaling_factor=a.mtp_loss_scaling_factor,
        mtp_only_training=a.mtp_only_training,
        opd_kl_coef=float(a.opd_kl_coef) if getattr(a, "opd_type", None) else 0.0,
        opd_only_reward=bool(a.opd_only_reward) and bool(getattr(a, "opd_type", None)),
        opd_kl_type=a.opd_kl_type, opd_jsd_alpha=a.opd_jsd_alpha, opd_norm_mode=a.opd_norm_mode,
        opd_log_prob_min_clamp=a.opd_log_prob_min_clamp, opd_per_token_clip=a.opd_per_token_clip,
        opd_token_selection={"student_sampled": "sampled_token"}.get(a.opd_token_selection, a.opd_token_selection),
        opd_log_prob_top_k=int(a.opd_log_prob_top_k or 0), use_routing_replay=bool(getattr(a, "use_routing_replay", False)),
        use_rollout_routing_replay=bool(getattr(a, "use_rollout_routing_replay", False) or getattr(a, "engine_return_routed_experts", False)),
        freeze_params_name_list=_freeze_list(a), problem_type=getattr(a, "problem_type", None),
        use_rollout_entropy=bool(getattr(a, "use_rollout_entropy", False)),
        compute_advantages_and_returns=not getattr(a, "disable_compute_advantages_and_returns", False),
        classification_threshold=float(getattr(a, "classification_threshold", 0.5) or 0.5),
        only_train_params_name_list=getattr(a, "only_train_params_name_list", None), loss=loss, optim=optim,
        ci=_ci_config(a), cp_attention="allgather" if getattr(a, "allgather_cp", False) else None)
