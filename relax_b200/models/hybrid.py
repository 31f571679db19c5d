"""Token mixers other than softmax attention, behind the interface of :class:`~relax_b200.models.transformer.Attention`,
so one decoder stack covers the hybrid families: Qwen3-Next (three GDN layers for every full-attention layer) and
GLM-MoE-DSA (sparse MLA attention with a lightning indexer in every layer).

Both run on the PyTorch ops of :mod:`relax_b200.models.gdn` / :mod:`relax_b200.models.dsa`; they need ``tp = cp = 1``
(their heads are not sharded yet) and are served by the trainer only - the rollout engine refuses these configs.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .dsa import DSAAttention
from .gdn import GatedDeltaNet


def _norm_holder(cfg, dtype, device):
    m = nn.Module()
    m.layer_norm_weight = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
    return m


class GDNMixer(nn.Module):
    def __init__(self, cfg, ps, dtype, device, gen, layer_idx):
        super().__init__()
        assert ps.tp.size == 1 and ps.cp.size == 1, "GDN layers: tp = cp = 1"
        self.linear_qkv = _norm_holder(cfg, dtype, device)     # the input norm lives where Attention keeps it
        self.gdn = GatedDeltaNet(cfg.hidden_size, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim, cfg.gdn_head_dim,
                                 eps=cfg.rms_norm_eps, dtype=dtype, device=device, seed=gen.seed * 1009 + layer_idx)

    def forward(self, x_normed, cos, sin, cu_seqlens, attn_fn=None, max_seqlen=None):
        assert cu_seqlens is not None and attn_fn is None
        return self.gdn(x_normed, cu_seqlens)


class DSAMixer(nn.Module):
    def __init__(self, cfg, ps, dtype, device, gen, layer_idx):
        super().__init__()
        assert ps.tp.size == 1 and ps.cp.size == 1, "DSA layers: tp = cp = 1"
        self.linear_qkv = _norm_holder(cfg, dtype, device)
        self.dsa = DSAAttention(cfg.hidden_size, cfg.num_attention_heads, cfg.dsa_q_lora, cfg.dsa_kv_lora, cfg.dsa_nope,
                                cfg.dsa_rope, cfg.dsa_v_head, cfg.dsa_index_heads, cfg.dsa_index_dim, cfg.dsa_topk,
                                cfg.rope_theta, cfg.rms_norm_eps, seed=gen.seed * 1013 + layer_idx, dtype=dtype, device=device)
        self.positions = None            # set by GPTModel.forward before the layer loop
        self.indexer_loss = None         # KL of the last forward in training mode (added to the loss by the trainer)

    def forward(self, x_normed, cos, sin, cu_seqlens, attn_fn=None, max_seqlen=None):
        assert cu_seqlens is not None and attn_fn is None and self.positions is not None
        self.indexer_loss = None
        if self.dsa.topk <= 0:
            return self.dsa(x_normed, self.positions, cu_seqlens, dense=True)
        if torch.is_grad_enabled():
            y, self.indexer_loss, _ = self.dsa(x_normed, self.positions, cu_seqlens, return_aux=True)
            return y
        return self.dsa(x_normed, self.positions, cu_seqlens)


def mixer_kind(cfg, layer_idx: int) -> str:
    if cfg.dsa_topk > 0 or cfg.multi_latent_attention:
        return "dsa"      # the same module; without a top-k it attends densely (plain MLA) and has no indexer loss
    if cfg.linear_attention_freq > 0 and (layer_idx + 1) % cfg.linear_attention_freq != 0:
        return "gdn"
    return "attention"


def collect_indexer_loss(model):
    """Sum of the DSA layers' indexer losses of the last forward (None when the model has none)."""
    terms = [m.indexer_loss for m in model.modules() if isinstance(m, DSAMixer) and m.indexer_loss is not None]
    return sum(terms) if terms else None
