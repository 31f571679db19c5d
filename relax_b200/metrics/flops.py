"""Model FLOPs accounting and MFU.

Counts the matrix-multiply FLOPs of one forward pass over a packed batch from the
model configuration (attention with the causal half, GQA projections, dense or MoE MLP with only
the routed experts, LM head), the way the reference's counter does for Megatron models
(relax/utils/training/flops_counter.py); backward is twice the forward, recomputation adds
another forward of the recomputed part.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Optional

from ..models.config import ModelConfig


@dataclass
class FlopsBreakdown:
    attn_proj: float = 0.0
    attn_core: float = 0.0
    mlp: float = 0.0
    router: float = 0.0
    lm_head: float = 0.0

    @property
    def total(self) -> float:
        return self.attn_proj + self.attn_core + self.mlp + self.router + self.lm_head


def forward_flops(cfg: ModelConfig, seq_lens: Iterable[int], lm_head_tokens: Optional[int] = None,
                  causal: bool = True) -> FlopsBreakdown:
    """FLOPs (multiply-add = 2) of one forward pass over sequences of the given lengths."""
    seq_lens = list(seq_lens)
    T = sum(seq_lens)
    h, hd = cfg.hidden_size, cfg.head_dim
    nq, nkv = cfg.num_attention_heads, cfg.num_query_groups
    L = cfg.num_layers
    b = FlopsBreakdown()
    b.attn_proj = L * 2.0 * T * h * (nq * hd + 2 * nkv * hd + nq * hd)
    sq = sum(s * s for s in seq_lens)
    b.attn_core = L * 4.0 * sq * nq * hd * (0.5 if causal else 1.0)
    n_moe = L if getattr(cfg, "num_experts", 0) else 0   # every layer is MoE in the supported MoE families
    n_dense = L - n_moe
    b.mlp = n_dense * 2.0 * T * h * cfg.ffn_hidden_size * 3
    if n_moe:
        b.mlp += n_moe * 2.0 * T * h * cfg.moe_ffn_hidden_size * 3 * cfg.moe_top_k
        b.router = n_moe * 2.0 * T * h * cfg.num_experts
        if getattr(cfg, "moe_shared_expert_size", 0):
            b.mlp += n_moe * 2.0 * T * h * cfg.moe_shared_expert_size * 3
    b.lm_head = 2.0 * (T if lm_head_tokens is None else lm_head_tokens) * h * cfg.vocab_size
    return b


def train_step_flops(cfg: ModelConfig, seq_lens: Iterable[int], lm_head_tokens: Optional[int] = None,
                     forward_only_passes: int = 0, recompute: bool = False) -> float:
    """One optimizer micro-step: forward + backward (2x) (+ a recomputed forward), plus
    ``forward_only_passes`` extra forwards (old-policy / reference log-probs in RL)."""
    f = forward_flops(cfg, seq_lens, lm_head_tokens).total
    return f * (3.0 + (1.0 if recompute else 0.0) + forward_only_passes)


def mfu(flops: float, seconds: float, n_gpus: int, peak_tflops_per_gpu: float) -> float:
    """Model FLOPs utilisation against a per-GPU dense peak given in TFLOP/s."""
    if seconds <= 0 or n_gpus <= 0 or peak_tflops_per_gpu <= 0:
        return 0.0
    return flops / seconds / (n_gpus * peak_tflops_per_gpu * 1e12)


B200_BF16_DENSE_TFLOPS = 2250.0
