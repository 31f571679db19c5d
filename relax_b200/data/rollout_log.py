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


def _flat(val, device=None):
    """Concatenate per-sample token-level values (tensors or lists of numbers) into one fp32 vector + lengths."""
    if torch.is_tensor(val[0]):
        lens = [int(v.numel()) for v in val]
        return torch.cat([v.reshape(-1).float() for v in val]), lens
    lens = [len(v) for v in val]
    t = torch.tensor([y for v in val for y in v], dtype=torch.float32)
    return (t.to(device) if device is not None else t), lens


def log_rollout_data(batch: dict, dp_group=None, device="cpu") -> dict:
    masks = batch.get("loss_masks")
    resp = batch.get("response_lengths")
    sums: dict = {}
    pending: dict = {}        # key -> 0-d device tensor (sum over samples of the per-sample masked mean), read once at the end
    mask_flat = mask_lens = seg = msum = None
    for key, val in batch.items():
        if key in SKIP or not isinstance(val, (list, tuple)) or len(val) == 0:
            continue
        first = val[0]
        if torch.is_tensor(first) and first.dim() == 0:
            pending[key] = torch.stack([x.float() for x in val]).sum()
            sums[key] = (None, len(val))
        elif torch.is_tensor(first) or (isinstance(first, (list, tuple)) and first and isinstance(first[0], (int, float))):
            # token level: masked mean inside each sample, then the mean over samples - a handful of kernels per
            # field over the concatenated samples (segment sums), not a handful per sample
            flat, lens = _flat(val)
            n = len(val)
            use_mask = masks is not None and resp is not None and lens == [int(r) for r in resp]
            if use_mask:
                if mask_flat is None or mask_flat.device != flat.device:
                    mask_flat, mask_lens = _flat(masks, flat.device)
                    mask_flat = mask_flat.to(flat.device)
                    seg = torch.repeat_interleave(torch.arange(n, device=flat.device),
                                                  torch.tensor(mask_lens, device=flat.device))
                    msum = torch.zeros(n, device=flat.device).index_add_(0, seg, mask_flat).clamp_min(1)
                per = torch.zeros(n, device=flat.device).index_add_(0, seg, flat * mask_flat) / msum
            else:
                sg = torch.repeat_interleave(torch.arange(n, device=flat.device), torch.tensor(lens, device=flat.device))
                cnt = torch.tensor(lens, dtype=torch.float32, device=flat.device).clamp_min(1)
                per = torch.zeros(n, device=flat.device).index_add_(0, sg, flat) / cnt
            pending[key] = per.sum()
            sums[key] = (None, n)
        elif isinstance(first, (int, float, bool)):
            sums[key] = (float(sum(float(x) for x in val)), len(val))
    if pending:
        keys_p = sorted(pending)
        dev0 = pending[keys_p[0]].device
        vals = torch.stack([pending[k].to(dev0) for k in keys_p]).tolist()      # ONE device read for all fields
        for k, v in zip(keys_p, vals):
            sums[k] = (float(v), sums[k][1])
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
