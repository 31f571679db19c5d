"""Samples -> train batch, and the per-row metadata the data plane keeps.

Counterpart of relax/utils/utils.py:96-177 (``convert_samples_to_train_data``
and the ``{total_lengths, sample_index}`` custom meta).
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..algo.ppo_utils import post_process_rewards
from ..types import Sample, SampleStatus


def convert_samples_to_train_data(samples: Sequence[Sample], *, advantage_estimator: str = "grpo",
                                  n_samples_per_prompt: int = 1, rewards_normalization: bool = True,
                                  grpo_std_normalization: bool = True, reward_key=None,
                                  custom_reward_post_process=None) -> dict:
    """``samples`` must be group-major (all samples of a prompt adjacent)."""
    raw = [s.get_reward_value(reward_key) for s in samples]
    if custom_reward_post_process is not None:
        raw_t, shaped = custom_reward_post_process(samples)
    else:
        raw_t = torch.tensor(raw, dtype=torch.float32)
        shaped = post_process_rewards(raw_t, n_samples_per_prompt, advantage_estimator,
                                      rewards_normalization, grpo_std_normalization)
    loss_masks = []
    for s in samples:
        m = s.loss_mask if s.loss_mask is not None else [1] * s.response_length
        if len(m) != s.response_length:
            raise ValueError(f"sample {s.index}: loss mask has {len(m)} entries for {s.response_length} response tokens")
        if s.remove_sample:
            m = [0] * s.response_length
        loss_masks.append(list(m))
    # rows that belong to the same logical sample share the denominator of the per-sample mean
    sums: dict = {}
    for s, m in zip(samples, loss_masks):
        sums[s.index] = sums.get(s.index, 0) + sum(m)
    batch = {
        "tokens": [list(s.tokens) for s in samples],
        "response_lengths": [s.response_length for s in samples],
        "rewards": shaped.tolist(),
        "raw_reward": raw,
        "group_index": [s.group_index for s in samples],
        "truncated": [1 if s.status == SampleStatus.TRUNCATED else 0 for s in samples],
        "sample_indices": [s.index for s in samples],
        "loss_masks": loss_masks,
        "sample_index_mask_sums": [sums[s.index] for s in samples],
        "total_lengths": [len(s.tokens) for s in samples],
        "weight_versions": [list(s.weight_versions) for s in samples],
    }
    if all(s.rollout_log_probs is not None for s in samples) and samples:
        batch["rollout_log_probs"] = [list(s.rollout_log_probs) for s in samples]
    if any(s.rollout_routed_experts is not None for s in samples):
        batch["rollout_routed_experts"] = [s.rollout_routed_experts for s in samples]
    if any(s.multimodal_train_inputs for s in samples):
        batch["multimodal_train_inputs"] = [s.multimodal_train_inputs for s in samples]
    if any(s.custom_advantage is not None for s in samples):
        # advantages set by user code (agentic exports): they replace the estimator's, one scalar per sample
        if not all(s.custom_advantage is not None or s.remove_sample for s in samples):
            raise ValueError("custom advantages must be set on every sample of the batch (or on none)")
        batch["custom_advantages"] = [float(s.custom_advantage or 0.0) for s in samples]
    if any(s.teacher_log_probs is not None for s in samples):
        batch["teacher_log_probs"] = [s.teacher_log_probs for s in samples]
    if any(s.metadata for s in samples):
        batch["metadata"] = [s.metadata for s in samples]
    return batch


def custom_meta_rows(batch: dict) -> list:
    return [{"total_lengths": tl, "sample_index": si} for tl, si in zip(batch["total_lengths"], batch["sample_indices"])]


def batch_num_rows(batch: dict) -> int:
    return len(batch["tokens"])
