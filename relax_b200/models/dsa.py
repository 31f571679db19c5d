"""DeepSeek-style sparse attention (DSA) for the GLM-MoE-DSA family: the lightning indexer that scores every
earlier token for every query, top-k selection, and multi-head latent attention (MLA, absorbed form) over the
selected latent KV rows only.

Covers the reference's tilelang ops (relax/models/glm_moe_dsa/ops/: ``tilelang_indexer_fwd.py`` indexer logits +
range cleaning, ``tilelang_indexer_bwd.py``, ``tilelang_sparse_mla_fwd.py`` / ``..._bwd.py``) and the attention
module that uses them (relax/models/glm_moe_dsa/dsa_attention.py: absorbed query/key :412-583, forward
:147-234).  The ops here are PyTorch (differentiable by autograd, chunked over queries so the gathered
``[rows, topk, 576]`` block stays bounded); they define the semantics and serve as the oracle.  There is no
hand-written sm_100a kernel for them yet.

Shapes follow the reference: the latent KV row is ``[kv_lora (512) | rope (64)]``, shared by all heads (MQA in
latent space); the absorbed query is ``[H, 576]``; the output is the ``[H, 512]`` latent mix, expanded per head
by the value up-projection afterwards.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops

NEG_INF = float("-inf")


def indexer_logits(q_idx, k_idx, head_w, starts, ends):
    """``logits[s, t] = sum_h head_w[s, h] * relu(q_idx[s, h] . k_idx[t])`` for ``starts[s] <= t < ends[s]``,
    ``-inf`` elsewhere.  ``q_idx [S, Hi, D]``, ``k_idx [Skv, D]``, ``head_w [S, Hi]`` -> fp32 ``[S, Skv]``."""
    s = torch.einsum("shd,td->sht", q_idx.float(), k_idx.float())
    logits = (F.relu(s) * head_w.float()[..., None]).sum(1)
    t = torch.arange(k_idx.shape[0], device=q_idx.device)[None, :]
    inside = (t >= starts[:, None]) & (t < ends[:, None])
    return logits.masked_fill(~inside, NEG_INF)


def topk_indices(logits, topk: int):
    """Indices of the ``topk`` largest finite logits per row, ``-1`` where a row has fewer candidates."""
    k = min(topk, logits.shape[1])
    # equal scores (the same token at two positions has the same indexer key): the earlier position wins, so that every
    # implementation of the selection - packed training rows, the rollout engine's per-request cache - picks the same set
    val, idx = logits.sort(dim=-1, descending=True, stable=True)
    val, idx = val[:, :k], idx[:, :k]
    idx = torch.where(torch.isfinite(val), idx, torch.full_like(idx, -1))
    if k < topk:
        idx = F.pad(idx, (0, topk - k), value=-1)
    return idx


def sparse_mla_attention(q, kv, idx, d_v: int = 512, scale: Optional[float] = None, rows_per_chunk: int = 256):
    """Attention of every query over its selected KV rows.  ``q [S, H, D]`` (absorbed, ``D = d_v + rope``),
    ``kv [Skv, D]``, ``idx [S, K]`` (``-1`` = empty slot).  Returns ``(out [S, H, d_v], lse [S, H])``; a query with
    no valid slot gets zeros and ``lse = -inf``."""
    S, H, D = q.shape
    scale = scale if scale is not None else D ** -0.5
    outs, lses = [], []
    for a in range(0, S, rows_per_chunk):
        qi, ii = q[a:a + rows_per_chunk].float(), idx[a:a + rows_per_chunk]
        valid = ii >= 0
        g = kv[ii.clamp_min(0)].float()                                 # [s, K, D]
        sc = torch.einsum("shd,skd->shk", qi, g) * scale
        sc = sc.masked_fill(~valid[:, None, :], NEG_INF)
        lse = torch.logsumexp(sc, -1)
        p = torch.exp(sc - torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))[..., None])
        p = torch.where(valid[:, None, :], p, torch.zeros_like(p))
        outs.append(torch.einsum("shk,skd->shd", p, g[..., :d_v]))
        lses.append(lse)
    return torch.cat(outs).to(q.dtype), torch.cat(lses)


def dense_mla_attention(q, kv, starts, ends, d_v: int = 512, scale: Optional[float] = None):
    """Every key in ``[starts, ends)``: what the sparse op computes when ``topk`` covers the whole range."""
    S, H, D = q.shape
    scale = scale if scale is not None else D ** -0.5
    sc = torch.einsum("shd,td->sht", q.float(), kv.float()) * scale
    t = torch.arange(kv.shape[0], device=q.device)[None, :]
    inside = (t >= starts[:, None]) & (t < ends[:, None])
    sc = sc.masked_fill(~inside[:, None, :], NEG_INF)
    p = torch.softmax(sc, -1)
    return torch.einsum("sht,td->shd", p, kv.float()[:, :d_v]).to(q.dtype), p


def indexer_kl_loss(idx_logits, attn_probs, idx):
    """Training signal of the indexer: KL(target || indexer) over the selected slots, where the target is the main
    attention's probability summed over heads and renormalised on the selected set (both detached from the trunk
    by the caller).  ``idx_logits [S, Skv]``, ``attn_probs [S, H, Skv]``, ``idx [S, K]``."""
    valid = idx >= 0
    j = idx.clamp_min(0)
    tgt = attn_probs.sum(1).gather(1, j) * valid
    tgt = tgt / tgt.sum(-1, keepdim=True).clamp_min(1e-20)
    lg = idx_logits.gather(1, j).masked_fill(~valid, NEG_INF)
    logp = torch.log_softmax(lg, -1)
    term = torch.where(tgt > 0, tgt * (torch.log(tgt.clamp_min(1e-20)) - logp), torch.zeros_like(tgt))
    rows = valid.any(-1)
    return term.sum(-1)[rows].mean() if rows.any() else idx_logits.sum() * 0.0


def causal_ranges(cu_seqlens, total: int):
    """Per packed row ``(start of its sequence, row + 1)``: the causal key range inside the row's own sequence."""
    rows = torch.arange(total, device=cu_seqlens.device)
    cu = cu_seqlens.to(torch.int64)
    seq = torch.bucketize(rows, cu[1:], right=True).clamp_max(cu.numel() - 2)
    return cu[:-1][seq], rows + 1


class DSAAttention(nn.Module):
    """MLA with the absorbed formulation plus the lightning indexer.

    ``q``: hidden -> ``q_lora`` -> norm -> per head ``[nope | rope]``; the ``nope`` part is carried into latent space
    with the key up-projection (``W_uk``), giving the ``[H, kv_lora + rope]`` query.  ``kv``: hidden ->
    ``[kv_lora | rope]`` latent row (norm on the latent part, RoPE on the tail), shared by all heads.  The indexer has
    its own small query heads, one key per token and per-head mixing weights, all read from the hidden state."""

    def __init__(self, hidden: int, heads: int, q_lora: int = 64, kv_lora: int = 32, nope: int = 16, rope: int = 8, v_head: int = 16,
                 idx_heads: int = 4, idx_dim: int = 16, topk: int = 16, rope_theta: float = 1e4, eps: float = 1e-6, seed: int = 0,
                 dtype=torch.float32, device="cpu"):
        super().__init__()
        self.H, self.nope, self.rope, self.kvl, self.vh, self.topk, self.eps, self.theta = heads, nope, rope, kv_lora, v_head, topk, eps, rope_theta
        self.Hi, self.Di = idx_heads, idx_dim
        gen = torch.Generator().manual_seed(seed)
        mk = lambda *s: nn.Parameter((torch.randn(*s, generator=gen) * 0.05).to(device=device, dtype=dtype))
        one = lambda n: nn.Parameter(torch.ones(n, dtype=dtype, device=device))
        self.linear_q_down_proj, self.linear_q_up_proj = nn.Module(), nn.Module()
        self.linear_q_down_proj.weight = mk(q_lora, hidden)
        self.linear_q_up_proj.weight = mk(heads * (nope + rope), q_lora)
        self.linear_q_up_proj.layer_norm_weight = one(q_lora)
        self.linear_kv_down_proj, self.linear_kv_up_proj = nn.Module(), nn.Module()
        self.linear_kv_down_proj.weight = mk(kv_lora + rope, hidden)
        self.linear_kv_up_proj.weight = mk(heads * (nope + v_head), kv_lora)      # per head [W_uk ; W_uv]
        self.linear_kv_up_proj.layer_norm_weight = one(kv_lora)
        self.linear_proj = nn.Module()
        self.linear_proj.weight = mk(hidden, heads * v_head)
        if topk <= 0:        # plain (dense) MLA: no indexer
            return
        self.indexer = nn.Module()
        self.indexer.linear_wq = nn.Module()
        self.indexer.linear_wq.weight = mk(idx_heads * idx_dim, hidden)
        self.indexer.linear_wk = nn.Module()
        self.indexer.linear_wk.weight = mk(idx_dim, hidden)
        self.indexer.linear_weights = nn.Module()
        self.indexer.linear_weights.weight = mk(idx_heads, hidden)

    def _rope(self, x, positions):
        cos, sin = ops.rope_cos_sin(positions, self.rope, self.theta, None)
        return ops.apply_rope(x, cos, sin)

    def absorbed_qkv(self, x, positions):
        T, H = x.shape[0], self.H
        ql = ops.rmsnorm(ops.linear(x, self.linear_q_down_proj.weight), self.linear_q_up_proj.layer_norm_weight, self.eps)
        q = ops.linear(ql, self.linear_q_up_proj.weight).view(T, H, self.nope + self.rope)
        q_nope, q_rope = q[..., : self.nope], self._rope(q[..., self.nope:].contiguous(), positions)
        kvd = ops.linear(x, self.linear_kv_down_proj.weight)
        c = ops.rmsnorm(kvd[:, : self.kvl].contiguous(), self.linear_kv_up_proj.layer_norm_weight, self.eps)
        k_rope = self._rope(kvd[:, None, self.kvl:].contiguous(), positions)[:, 0]
        w = self.linear_kv_up_proj.weight.view(H, self.nope + self.vh, self.kvl)
        w_uk, w_uv = w[:, : self.nope], w[:, self.nope:]
        q_abs = torch.einsum("thn,hnc->thc", q_nope.float(), w_uk.float()).to(x.dtype)
        return torch.cat([q_abs, q_rope], -1), torch.cat([c, k_rope], -1), w_uv

    def forward(self, x, positions, cu_seqlens, return_aux: bool = False, dense: bool = False):
        T = x.shape[0]
        q, kv, w_uv = self.absorbed_qkv(x, positions)
        starts, ends = causal_ranges(cu_seqlens, T)
        scale = (self.nope + self.rope) ** -0.5
        if dense and not return_aux:
            lat, _ = dense_mla_attention(q, kv, starts, ends, self.kvl, scale)
            o = torch.einsum("thc,hvc->thv", lat.float(), w_uv.float()).to(x.dtype).reshape(T, self.H * self.vh)
            return ops.linear(o, self.linear_proj.weight)
        xd = x.detach()        # the indexer learns from its own loss only
        lg = indexer_logits(ops.linear(xd, self.indexer.linear_wq.weight).view(T, self.Hi, self.Di),
                            ops.linear(xd, self.indexer.linear_wk.weight), ops.linear(xd, self.indexer.linear_weights.weight) * self.Hi ** -0.5,
                            starts, ends)
        idx = topk_indices(lg.detach(), self.topk)
        if dense:
            lat, _ = dense_mla_attention(q, kv, starts, ends, self.kvl, scale)
        else:
            lat, _ = sparse_mla_attention(q, kv, idx, self.kvl, scale)
        o = torch.einsum("thc,hvc->thv", lat.float(), w_uv.float()).to(x.dtype).reshape(T, self.H * self.vh)
        y = ops.linear(o, self.linear_proj.weight)
        if not return_aux:
            return y
        with torch.no_grad():
            _, probs = dense_mla_attention(q, kv, starts, ends, self.kvl, scale)
        return y, indexer_kl_loss(lg, probs, idx), idx
