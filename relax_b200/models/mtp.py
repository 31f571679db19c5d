"""Multi-token prediction (MTP) head: extra depth-k blocks that predict token ``t+k+1`` from the trunk's
hidden state at ``t`` and the embedding of token ``t+k``, sharing the embedding and the LM head.

Covers the reference's MTP training switches (relax/utils/arguments.py MTP group :2585-2617:
``--enable-mtp-training``, ``--mtp-num-layers``, ``--mtp-loss-scaling-factor``) and the MTP-only loss
(relax/backends/megatron/loss.py mtp_only_loss_function :1431).  Block layout follows Megatron-core's
``MultiTokenPredictionLayer`` parameter names (``enorm``, ``hnorm``, ``eh_proj``, ``transformer_layer``,
``final_layernorm``) so the checkpoint name tables apply.

Each block works on the packed token stream of the trunk: tokens are shifted left *inside* their own
sequence (no token crosses a ``cu_seqlens`` boundary), rows whose shifted token or target falls outside the
sequence are reported as invalid, and the same varlen attention runs over the same boundaries.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..parallel import tp as TP


def shift_in_sequence(tokens: torch.Tensor, cu_seqlens: torch.Tensor, k: int):
    """``out[i] = tokens[i + k]`` when row ``i + k`` belongs to the sequence of row ``i``, else 0;
    also returns the boolean validity of every row."""
    T = tokens.numel()
    rows = torch.arange(T, device=tokens.device)
    cu = cu_seqlens.to(torch.int64)
    seq = torch.bucketize(rows, cu[1:], right=True).clamp_max(cu.numel() - 2)
    end = cu[1:][seq]
    ok = rows + k < end
    src = torch.where(ok, rows + k, rows)
    return torch.where(ok, tokens[src], torch.zeros_like(tokens)), ok


class MTPBlock(nn.Module):
    def __init__(self, cfg, ps, dtype, device, gen, depth: int):
        super().__init__()
        from .transformer import TransformerLayer

        self.cfg, self.ps, self.depth = cfg, ps, depth
        H = cfg.hidden_size
        for name in ("enorm", "hnorm", "final_layernorm"):
            m = nn.Module()
            m.weight = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
            m.weight.tp_replicated = True
            setattr(self, name, m)
        self.eh_proj = nn.Module()
        self.eh_proj.weight = nn.Parameter(gen.draw(f"mtp.{depth}.eh_proj", (H, 2 * H), 0.02).to(device=device, dtype=dtype))
        self.eh_proj.weight.tp_replicated = True   # small [H, 2H]; kept whole on every TP rank
        self.transformer_layer = TransformerLayer(cfg, ps, dtype, device, gen, cfg.num_layers + depth)

    def forward(self, h_prev, emb, cos, sin, cu_seqlens, max_seqlen=None):
        """``h_prev`` / ``emb``: the sequence-parallel shard ``[T / tp, H]``.  Returns the block's un-normalised
        output (input of the next depth) and its normalised output (input of the shared LM head)."""
        eps = self.cfg.rms_norm_eps
        x = torch.cat([ops.rmsnorm(emb, self.enorm.weight, eps), ops.rmsnorm(h_prev, self.hnorm.weight, eps)], -1)
        h = ops.linear(x, self.eh_proj.weight)
        h = self.transformer_layer(h, cos, sin, cu_seqlens, None, max_seqlen)
        return h, ops.rmsnorm(h, self.final_layernorm.weight, eps)


def mtp_forward(model, prenorm_hidden, tokens, positions, cu_seqlens, rows, max_seqlen=None):
    """Run every MTP depth.  ``prenorm_hidden`` is the trunk's last-layer output before the final norm
    (sequence-parallel shard).  ``rows`` are the packed rows whose main-head target is trained (row ``r``
    predicts token ``r + 1``); for depth ``k`` the block at row ``r`` predicts token ``r + k + 1``.

    Returns a list of ``(log_probs[len(rows)], valid[len(rows)])`` per depth; ``valid`` is False where the
    shifted token or the target lies outside the row's sequence."""
    sp = model.sequence_parallel
    cos, sin = model.rope_tables(positions)
    out, h = [], prenorm_hidden
    for k, block in enumerate(model.mtp.layers, start=1):
        tok_k, ok_in = shift_in_sequence(tokens, cu_seqlens, k)
        tgt_k, ok_tgt = shift_in_sequence(tokens, cu_seqlens, k + 1)
        emb = model.embedding.word_embeddings(tok_k, sp)
        h, hn = block(h, emb, cos, sin, cu_seqlens, max_seqlen)
        if sp:
            hn = TP.gather_seq(hn, model.ps.tp)
        lp, _ = model.log_probs(hn.index_select(0, rows), tgt_k.index_select(0, rows), 1.0, False)
        out.append((lp, (ok_in & ok_tgt).index_select(0, rows)))
    return out
