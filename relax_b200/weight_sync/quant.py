"""Quantisation hooks of the weight sync: what the rollout engine serves can be the trainer's bf16
weights passed through the serving format's quantiser (block-scaled fp8 e4m3 with fp32 or
power-of-two ``ue8m0`` scales, or grouped int4), so rollout log-probs already carry the
quantisation error the deployed model will have (relax/backends/megatron/weight_conversion/
processors/quantizer_fp8.py, quantizer_compressed_tensors.py; the int4 path is the reference's
only in-tree CUDA kernel, relax/backends/megatron/kernels/int4_qat).  The sm_100a kernels are in
csrc/elementwise.cu; the statements in ops/reference.py.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from .. import ops

_SKIP = ("norm", "embed", "lm_head", "router", "bias")


def _eligible(name: str, t: torch.Tensor) -> bool:
    return t.dim() == 2 and not any(k in name for k in _SKIP)


def fp8_roundtrip(block: int = 128, ue8m0: bool = False) -> Callable:
    def fn(name: str, w: torch.Tensor) -> torch.Tensor:
        if not _eligible(name, w):
            return w
        q, scale_inv = ops.blockwise_cast_to_fp8(w, block, ue8m0)
        return ops.blockwise_dequant_fp8(q, scale_inv, block, w.dtype)

    return fn


def int4_roundtrip(group: int = 128, sym: bool = True) -> Callable:
    def fn(name: str, w: torch.Tensor) -> torch.Tensor:
        if not _eligible(name, w) or w.shape[1] % group:
            return w
        return ops.fake_int4_quant(w, 1, group, sym)[0]

    return fn


def make_hook(kind: Optional[str], **kw) -> Optional[Callable]:
    if not kind or kind == "none":
        return None
    if kind == "fp8":
        return fp8_roundtrip(**kw)
    if kind == "int4":
        return int4_roundtrip(**kw)
    raise ValueError(f"unknown weight-sync quantisation {kind!r} (fp8, int4, none)")
