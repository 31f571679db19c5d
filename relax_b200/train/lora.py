"""LoRA adapters for the training model: wrap, train only the adapters, merge for weight sync,
export / import the adapter, merge into a full checkpoint.

The reference wraps Megatron modules through Megatron-Bridge PEFT (relax/backends/megatron/
model_provider.py:526-600), syncs either merged weights or the adapter itself to the rollout
engines (relax/distributed/checkpoint_service/backends/device_direct.py:1083-1268,
relax/backends/megatron/weight_update/lora_adapter_sync.py) and ships a merge tool
(scripts/tools/merge_lora_adapter_to_hf.py).  Here an adapted linear keeps its frozen weight
``W`` and adds ``scale * B (A x)`` with ``A [r, in]`` ~ N(0, 1/r) and ``B [out, r] = 0``; under
tensor parallelism ``A`` follows the input sharding of ``W`` and ``B`` its output sharding, and the
rank-``r`` intermediate is what crosses the collective (``r`` columns instead of the full width).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional, Tuple

import torch
import torch.nn as nn

from ..parallel import tp as TP

DEFAULT_TARGETS = ("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2")
_COLUMN_PARALLEL = ("linear_qkv", "linear_fc1")   # input: sequence shard (gathered), output: sharded features


@dataclass
class LoRAConfig:
    rank: int = 16
    alpha: float = 32.0
    target_modules: Tuple[str, ...] = DEFAULT_TARGETS
    seed: int = 1234
    dropout: float = 0.0          # on the adapter's input, while gradients are enabled (peft's lora_dropout)

    @property
    def scale(self) -> float:
        return self.alpha / self.rank


def _adapted_modules(model) -> Iterator[Tuple[str, nn.Module]]:
    for name, mod in model.named_modules():
        if hasattr(mod, "lora_A"):
            yield name, mod


def apply_lora(model, cfg: LoRAConfig) -> List[str]:
    """Freeze every existing parameter and attach adapters to the target linears.  Call BEFORE the optimizer
    is built.  Returns the adapted module names."""
    for p in model.parameters():
        p.requires_grad_(False)
    g = torch.Generator(device="cpu").manual_seed(cfg.seed)
    names = []
    for name, mod in list(model.named_modules()):
        leaf = name.rsplit(".", 1)[-1]
        if leaf not in cfg.target_modules or not hasattr(mod, "weight") or mod.weight.dim() != 2:
            continue
        w = mod.weight
        out_f, in_f = w.shape
        a = torch.randn(cfg.rank, in_f, generator=g) / math.sqrt(cfg.rank)
        mod.lora_A = nn.Parameter(a.to(device=w.device, dtype=w.dtype))
        mod.lora_B = nn.Parameter(torch.zeros(out_f, cfg.rank, device=w.device, dtype=w.dtype))
        mod.lora_scale = cfg.scale
        mod.lora_dropout = float(cfg.dropout)
        # the replicated factor sees a different token / feature shard on every TP rank: its gradient is a partial sum
        (mod.lora_A if leaf in _COLUMN_PARALLEL else mod.lora_B).tp_replicated = True
        names.append(name)
    model.lora_config = cfg
    return names


def lora_delta(mod, x, tp_group, column_parallel: bool):
    """``scale * B (A x)`` in the layout of the adapted linear's output.  ``x`` is the same tensor the base
    linear receives (a sequence shard for column-parallel layers, feature-sharded rows for row-parallel)."""
    if not hasattr(mod, "lora_A"):
        return None
    p_drop = getattr(mod, "lora_dropout", 0.0)
    if p_drop > 0.0 and torch.is_grad_enabled():
        x = torch.nn.functional.dropout(x, p_drop, training=True)
    xa = torch.nn.functional.linear(x, mod.lora_A)              # [rows, r]
    if column_parallel:
        xa = TP.gather_seq(xa, tp_group)                         # rows of every rank
    else:
        xa = TP.reduce_scatter_seq(xa, tp_group)                 # sum of the partial products, my rows
    return torch.nn.functional.linear(xa, mod.lora_B) * mod.lora_scale


def merged_weight(mod) -> torch.Tensor:
    """``W + scale * B A`` of this rank's shard (fp32 product, cast back)."""
    w = mod.weight
    if not hasattr(mod, "lora_A"):
        return w
    return (w.float() + mod.lora_scale * (mod.lora_B.float() @ mod.lora_A.float())).to(w.dtype)


def merged_named_params(model) -> List[Tuple[str, torch.Tensor]]:
    """``named_parameters`` of the equivalent plain model: adapter factors folded into the weights they adapt
    (what the merged-weights sync mode sends to the rollout engines)."""
    adapted = dict(_adapted_modules(model))
    out = []
    for n, p in model.named_parameters():
        if n.endswith(".lora_A") or n.endswith(".lora_B"):
            continue
        modname = n.rsplit(".", 1)[0]
        if n.endswith(".weight") and modname in adapted:
            out.append((n, merged_weight(adapted[modname])))
        else:
            out.append((n, p))
    return out


def adapter_state_dict(model) -> Dict[str, torch.Tensor]:
    return {n: p.detach().clone() for n, p in model.named_parameters() if n.endswith((".lora_A", ".lora_B"))}


def load_adapter_state_dict(model, sd: Dict[str, torch.Tensor]):
    own = dict(model.named_parameters())
    missing = [k for k in sd if k not in own]
    if missing:
        raise KeyError(f"adapter tensors without a matching module: {missing[:4]}")
    with torch.no_grad():
        for k, v in sd.items():
            own[k].copy_(v)


def adapter_fingerprint(model) -> float:
    """Cheap change detector for adapter-mode sync: only re-send an adapter whose factors moved."""
    return float(sum(p.detach().float().abs().sum() for n, p in model.named_parameters() if n.endswith(".lora_B")))


def merge_and_unload(model):
    """Fold the adapters into the base weights in place and remove them (export of a plain checkpoint)."""
    with torch.no_grad():
        for _, mod in list(_adapted_modules(model)):
            mod.weight.copy_(merged_weight(mod))
            del mod.lora_A, mod.lora_B
    for p in model.parameters():
        p.requires_grad_(True)
