"""Per-rollout summary metrics of a training batch (relax/backends/megatron/data.py log_rollout_data :957-1090).

Token-level fields (log-probs, advantages, returns, values, ... - one tensor of response length per sample) are
averaged per sample over the positions its loss mask keeps and then over samples; per-sample scalars (rewards,
lengths, truncation flags) are averaged directly; everything is reduced over the data-parallel group so every rank
reports the global value.  Keys come out as ``rollout/<field>``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

SKIP = {"tokens", "multimodal_train_inputs", "loss_masks", "sample_indices", "sample_index_mask_sums",
        "rollout_routed_experts", "max_seq_lens", "dynamic_global_batch_size", "metadata", "weight_versions", "prompt",
        "response", "label", "status", "group_index", "index"}


def log_rollout_data(batch: dict, dp_group=None, device="cpu") -> dict:
    masks = batch.get("loss_masks")
    resp = batch.get("response_lengths")
    sums: dict = {}
    for key, val in batch.items():
        if key in SKIP or not isinstance(val, (list, tuple)) or len(val) == 0:
            continue
        first = val[0]
        tot, cnt = 0.0, 0
        if torch.is_tensor(first) and first.dim() == 0:
            tot, cnt = float(torch.stack([x.float() for x in val]).sum()), len(val)
        elif torch.is_tensor(first) or (isinstance(first, (list, tuple)) and first and isinstance(first[0], (int, float))):
            # token level: masked mean inside each sample, then the mean over samples; the per-sample means stay
            # on the tensors' device and come to the host in one read per field
            means = []
            for i, v in enumerate(val):
                t = torch.as_tensor(v, dtype=torch.float32).reshape(-1)
                if masks is not None and resp is not None and t.numel() == int(resp[i]):
                    m = torch.as_tensor(masks[i], dtype=torch.float32, device=t.device).reshape(-1)
                    means.append((t * m).sum() / m.sum().clamp_min(1))
                elif t.numel():
                    means.append(t.mean())
                cnt += 1
            tot = float(torch.stack(means).sum()) if means else 0.0
        elif isinstance(first, (int, float, bool)):
            tot, cnt = float(sum(float(x) for x in val)), len(val)
        else:
            continue
        sums[key] = (tot, cnt)
    if resp is not None and batch.get("total_lengths") is not None:
        sums["prompt_lengths"] = (float(sum(int(t) - int(r) for t, r in zip(batch["total_lengths"], resp))), len(resp))
    keys = sorted(sums)
    vec = torch.tensor([x for k in keys for x in sums[k]], dtype=torch.float64, device=device)
    if dp_group is not None and dist.is_initialized() and dist.get_world_size(dp_group) > 1:
        # every replica holds the same fields (they depend on the configuration only)
        dist.all_reduce(vec, group=dp_group)
    out = {}
    for i, k in enumerate(keys):
        out[f"rollout/{k}"] = float(vec[2 * i] / vec[2 * i + 1].clamp_min(1))
    return out
