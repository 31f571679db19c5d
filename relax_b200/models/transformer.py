"""Qwen/Llama-style decoder on packed (thd) token streams, with TP/SP/CP/EP.

Parameter names and tensor layouts follow Megatron-core's GPT model with the
TransformerEngine layer spec, so checkpoints and the weight-conversion tables
(relax/backends/megatron/weight_conversion/qwen2.py, qwen3moe.py) apply:

* ``self_attention.linear_qkv.weight``: ``[ng * (q_per_group + 2) * hd, hidden]``
  interleaved per query group ``[q_0..q_{g-1}, k, v]``; TP shards whole groups.
* ``mlp.linear_fc1.weight``: ``[2 * ffn, hidden]`` as ``[gate; up]`` per TP shard.
* norms are fused into the following linear's name
  (``linear_qkv.layer_norm_weight``, ``linear_fc1.layer_norm_weight``).

The forward works on one packed micro-batch: ``tokens[T]``, ``cu_seqlens``,
``positions``.  With sequence parallelism the residual stream is sharded along
tokens (``T / tp`` rows per rank).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..parallel import tp as TP
from ..parallel.state import ParallelState, single_process_state
from .config import ModelConfig

_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


class ParamInit:
    """Per-parameter deterministic initialiser: each FULL (unsharded) tensor is
    drawn from a generator seeded by ``(seed, parameter name)`` on the target
    device, so every parallel layout and pipeline stage of the same seed holds
    the same model and no layout has to draw tensors it does not own."""

    def __init__(self, seed: int, device):
        self.seed, self.device = seed, torch.device(device)

    def draw(self, name: str, shape, std: float) -> torch.Tensor:
        import zlib

        g = torch.Generator(device=self.device)
        g.manual_seed((self.seed * 1000003 + zlib.crc32(name.encode())) % (2**63 - 1))
        w = torch.empty(shape, dtype=torch.float32, device=self.device)
        return w.normal_(0.0, std, generator=g)


def _lora():
    from ..train import lora

    return lora


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, ps: ParallelState, dtype, device, gen, layer_idx: int):
        super().__init__()
        self.cfg, self.ps, self.layer_idx = cfg, ps, layer_idx
        tp = ps.tp.size
        assert cfg.num_query_groups % tp == 0, "TP must divide the number of KV groups"
        self.ng = cfg.num_query_groups // tp
        self.qpg = cfg.num_attention_heads // cfg.num_query_groups
        hd = cfg.head_dim
        self.linear_qkv = nn.Module()
        self.linear_qkv.layer_norm_weight = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
        # draw the FULL weight so every TP layout of the same seed holds the same model
        # rows of one KV group: its query heads, (Qwen3.5 gated attention) one gate row per query feature, its key, its value
        self.gate = bool(cfg.attention_output_gate)
        self.grp = self.qpg * (2 if self.gate else 1) + 2
        full = gen.draw(f"layers.{layer_idx}.qkv", (cfg.num_query_groups * self.grp * hd, cfg.hidden_size), 0.02)
        rows = self.ng * self.grp * hd
        self.linear_qkv.weight = nn.Parameter(full[ps.tp.rank * rows:(ps.tp.rank + 1) * rows].to(device=device, dtype=dtype))
        if cfg.qkv_bias:
            self.linear_qkv.bias = nn.Parameter(torch.zeros(rows, dtype=dtype, device=device))
        fullo = gen.draw(f"layers.{layer_idx}.proj", (cfg.hidden_size, cfg.q_size), 0.02 / math.sqrt(2 * cfg.num_layers))
        cols = cfg.q_size // tp
        self.linear_proj = nn.Module()
        self.linear_proj.weight = nn.Parameter(fullo[:, ps.tp.rank * cols:(ps.tp.rank + 1) * cols].contiguous().to(device=device, dtype=dtype))
        if cfg.qk_layernorm:
            self.q_layernorm = nn.Module()
            self.q_layernorm.weight = nn.Parameter(torch.ones(hd, dtype=dtype, device=device))
            self.k_layernorm = nn.Module()
            self.k_layernorm.weight = nn.Parameter(torch.ones(hd, dtype=dtype, device=device))

    def split_qkv(self, qkv):
        T = qkv.shape[0]
        hd = self.cfg.head_dim
        x = qkv.view(T, self.ng, self.grp, hd)
        q = x[:, :, : self.qpg].reshape(T, self.ng * self.qpg, hd)
        k = x[:, :, self.grp - 2]
        v = x[:, :, self.grp - 1]
        if self.gate:
            self._gate = x[:, :, self.qpg: 2 * self.qpg].reshape(T, self.ng * self.qpg, hd)
        return q, k, v

    def _rope(self, x, cos, sin):
        rot = self.cfg.rotary_dim
        if rot >= self.cfg.head_dim:
            return ops.apply_rope(x, cos, sin)
        # partial rotary: only the first `rot` features of every head carry position
        return torch.cat([ops.apply_rope(x[..., :rot].contiguous(), cos, sin), x[..., rot:]], -1)

    def forward(self, x_normed, cos, sin, cu_seqlens, attn_fn=None, max_seqlen=None):
        cfg = self.cfg
        qkv = TP.ag_linear(x_normed, self.linear_qkv.weight, self.ps.tp)
        if hasattr(self.linear_qkv, "lora_A"):
            qkv = qkv + _lora().lora_delta(self.linear_qkv, x_normed, self.ps.tp, True)
        if cfg.qkv_bias:
            qkv = qkv + self.linear_qkv.bias
        q, k, v = self.split_qkv(qkv)
        if cfg.qk_layernorm:
            q = ops.rmsnorm(q, self.q_layernorm.weight, cfg.rms_norm_eps)
            k = ops.rmsnorm(k, self.k_layernorm.weight, cfg.rms_norm_eps)
        q = self._rope(q, cos, sin)
        k = self._rope(k, cos, sin)
        if attn_fn is not None:
            o = attn_fn(self.layer_idx, q, k, v)
        else:
            o = ops.attention_varlen(q, k, v.contiguous(), cu_seqlens, causal=True, max_seqlen=max_seqlen)
        if self.gate:        # Qwen3.5: attention output gated per feature by a sigmoid of the gate projection
            o = o * torch.sigmoid(self._gate.float()).to(o.dtype)
            self._gate = None
        o = o.reshape(o.shape[0], -1)
        y = TP.linear_rs(o, self.linear_proj.weight, self.ps.tp)
        if hasattr(self.linear_proj, "lora_A"):
            y = y + _lora().lora_delta(self.linear_proj, o, self.ps.tp, False)
        return y


class MLP(nn.Module):
    def __init__(self, cfg: ModelConfig, ps: ParallelState, dtype, device, gen, layer_idx: int = 0):
        super().__init__()
        self.cfg, self.ps = cfg, ps
        tp = ps.tp.size
        f = cfg.ffn_hidden_size
        assert f % tp == 0
        fl = f // tp
        full1 = gen.draw(f"layers.{layer_idx}.fc1", (2 * f, cfg.hidden_size), 0.02)
        r = ps.tp.rank
        w1 = torch.cat([full1[r * fl:(r + 1) * fl], full1[f + r * fl: f + (r + 1) * fl]], 0)
        self.linear_fc1 = nn.Module()
        self.linear_fc1.layer_norm_weight = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
        self.linear_fc1.weight = nn.Parameter(w1.to(device=device, dtype=dtype))
        full2 = gen.draw(f"layers.{layer_idx}.fc2", (cfg.hidden_size, f), 0.02 / math.sqrt(2 * cfg.num_layers))
        self.linear_fc2 = nn.Module()
        self.linear_fc2.weight = nn.Parameter(full2[:, r * fl:(r + 1) * fl].contiguous().to(device=device, dtype=dtype))

    def forward(self, x_normed):
        gu = TP.ag_linear(x_normed, self.linear_fc1.weight, self.ps.tp)
        if hasattr(self.linear_fc1, "lora_A"):
            gu = gu + _lora().lora_delta(self.linear_fc1, x_normed, self.ps.tp, True)
        a = ops.swiglu(gu)
        y = TP.linear_rs(a, self.linear_fc2.weight, self.ps.tp)
        if hasattr(self.linear_fc2, "lora_A"):
            y = y + _lora().lora_delta(self.linear_fc2, a, self.ps.tp, False)
        return y


class TransformerLayer(nn.Module):
    def __init__(self, cfg, ps, dtype, device, gen, layer_idx):
        super().__init__()
        self.cfg = cfg
        from .hybrid import DSAMixer, GDNMixer, mixer_kind

        kind = mixer_kind(cfg, layer_idx)
        mixer = {"attention": Attention, "gdn": GDNMixer, "dsa": DSAMixer}[kind]
        self.self_attention = mixer(cfg, ps, dtype, device, gen, layer_idx)
        if cfg.is_moe_layer(layer_idx):
            from .moe import MoEMLP

            self.mlp = MoEMLP(cfg, ps, dtype, device, gen, layer_idx)
            self.pre_mlp_layernorm = nn.Module()
            self.pre_mlp_layernorm.weight = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
            self.is_moe_layer = True
        else:
            self.mlp = MLP(cfg, ps, dtype, device, gen, layer_idx)
            self.is_moe_layer = False
        if cfg.sandwich_norm:
            one = lambda: nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
            self.post_self_attn_layernorm = nn.Module()
            self.post_self_attn_layernorm.weight = one()
            self.post_mlp_layernorm = nn.Module()
            self.post_mlp_layernorm.weight = one()

    def mlp_norm_weight(self):
        return self.pre_mlp_layernorm.weight if self.is_moe_layer else self.mlp.linear_fc1.layer_norm_weight

    def forward(self, h, cos, sin, cu_seqlens, attn_fn=None, max_seqlen=None):
        eps = self.cfg.rms_norm_eps
        x = ops.rmsnorm(h, self.self_attention.linear_qkv.layer_norm_weight, eps)
        a = self.self_attention(x, cos, sin, cu_seqlens, attn_fn, max_seqlen)
        if self.cfg.sandwich_norm:      # GLM-4: h += norm(attention(norm(h))); h += norm(mlp(norm(h)))
            a = ops.rmsnorm(a, self.post_self_attn_layernorm.weight, eps)
        x, h = ops.add_rmsnorm(a, h, self.mlp_norm_weight(), eps)
        m = self.mlp(x)
        if self.cfg.sandwich_norm:
            m = ops.rmsnorm(m, self.post_mlp_layernorm.weight, eps)
        return h + m


def _vocab_shard(gen, name, cfg, v_pad, start, v_local, dtype):
    full = gen.draw(name, (cfg.vocab_size, cfg.hidden_size), 0.02)
    if v_pad > cfg.vocab_size:
        full = torch.cat([full, full.new_zeros(v_pad - cfg.vocab_size, cfg.hidden_size)], 0)
    return full[start:start + v_local].to(dtype).contiguous()


class _EmbeddingLookup(torch.autograd.Function):
    """``weight[idx]`` (rows with ``keep`` false give zeros) whose backward adds the incoming rows straight into the
    optimizer's fp32 gradient buffer of the weight (``weight.main_grad``) instead of materialising a dense
    [vocab, hidden] gradient and adding that: per micro-batch only the rows that were looked up are touched."""

    @staticmethod
    def forward(ctx, weight, idx, keep):
        ctx.weight = weight
        ctx.save_for_backward(idx, keep if keep is not None else idx.new_empty(0))
        ctx.has_keep = keep is not None
        out = weight.detach()[idx]
        return out * keep[:, None].to(out.dtype) if keep is not None else out

    @staticmethod
    def backward(ctx, dy):
        idx, keep = ctx.saved_tensors
        w = ctx.weight
        if ctx.has_keep:
            dy = dy * keep[:, None].to(dy.dtype)
        mg = getattr(w, "main_grad", None)
        if mg is not None and mg.dtype == torch.float32 and w.grad is not mg:
            # sort-based accumulation: repeated tokens are summed in a fixed order (bit-identical reruns)
            mg.index_put_((idx,), dy.float(), accumulate=True)
            return None, None, None
        g = torch.zeros_like(w)
        g.index_put_((idx,), dy.to(g.dtype), accumulate=True)
        return g, None, None


class VocabParallelEmbedding(nn.Module):
    def __init__(self, cfg, ps, dtype, device, gen):
        super().__init__()
        self.ps = ps
        tp = ps.tp.size
        self.v_pad = (cfg.vocab_size + tp - 1) // tp * tp
        self.v_local = self.v_pad // tp
        self.start = ps.tp.rank * self.v_local
        self.weight = nn.Parameter(_vocab_shard(gen, "embedding", cfg, self.v_pad, self.start, self.v_local, dtype))

    def forward(self, tokens, sequence_parallel: bool):
        g = self.ps.tp
        if g.size == 1:
            return _EmbeddingLookup.apply(self.weight, tokens, None) if self.weight.requires_grad else self.weight[tokens]
        loc = tokens - self.start
        ok = (loc >= 0) & (loc < self.v_local)
        loc = torch.where(ok, loc, torch.zeros_like(loc))
        if self.weight.requires_grad:
            e = _EmbeddingLookup.apply(self.weight, loc, ok)
        else:
            e = self.weight[loc] * ok[:, None].to(self.weight.dtype)
        if sequence_parallel:
            return TP.reduce_scatter_seq(e, g)
        return TP.reduce_from_tp(e, g)


class GPTModel(nn.Module):
    """Decoder-only LM.  ``forward`` returns the final hidden states
    (sequence-parallel shard gathered back to all ``T`` rows); the LM head is
    applied by :meth:`log_probs` (fused with the loss) or :meth:`logits`."""

    def __init__(self, cfg: ModelConfig, ps: Optional[ParallelState] = None, device="cpu", seed: int = 0,
                 dtype: Optional[torch.dtype] = None, recompute: bool = False, pp_layers: Optional[range] = None):
        super().__init__()
        self.cfg = cfg
        self.ps = ps or single_process_state()
        self.dtype = dtype or _DTYPES[cfg.dtype]
        self.recompute = recompute
        self.sequence_parallel = self.ps.tp.size > 1
        gen = ParamInit(seed, device)
        ps_ = self.ps
        if pp_layers is None:
            per = cfg.num_layers // ps_.pp.size
            pp_layers = range(ps_.pp.rank * per, (ps_.pp.rank + 1) * per)
        self.pp_layers = pp_layers
        self.pre_process = ps_.is_pp_first
        self.post_process = ps_.is_pp_last
        tp = ps_.tp.size
        v_pad = (cfg.vocab_size + tp - 1) // tp * tp
        self.v_local, self.vocab_start = v_pad // tp, ps_.tp.rank * (v_pad // tp)
        if self.pre_process or (self.post_process and (cfg.tie_word_embeddings or cfg.mtp_num_layers > 0)):
            self.embedding = nn.Module()
            self.embedding.word_embeddings = VocabParallelEmbedding(cfg, ps_, self.dtype, device, gen)
        self.decoder = nn.Module()
        self.decoder.layers = nn.ModuleList(
            [TransformerLayer(cfg, ps_, self.dtype, device, gen, i) for i in pp_layers])
        if self.post_process:
            self.decoder.final_layernorm = nn.Module()
            self.decoder.final_layernorm.weight = nn.Parameter(torch.ones(cfg.hidden_size, dtype=self.dtype, device=device))
            if not cfg.tie_word_embeddings:
                self.output_layer = nn.Module()
                self.output_layer.weight = nn.Parameter(
                    _vocab_shard(gen, "output_layer", cfg, v_pad, self.vocab_start, self.v_local, self.dtype))
            if cfg.value_head:
                self.value_head = nn.Module()
                self.value_head.weight = nn.Parameter(torch.zeros(1, cfg.hidden_size, dtype=self.dtype, device=device))
            if cfg.num_classes > 0:
                self.score = nn.Module()
                self.score.weight = nn.Parameter(
                    gen.draw("score", (cfg.num_classes, cfg.hidden_size), 0.02).to(device=device, dtype=self.dtype))
                self.score.weight.tp_replicated = True
            if cfg.mtp_num_layers > 0:
                from .mtp import MTPBlock

                assert ps_.pp.size == 1 and ps_.cp.size == 1, "MTP blocks share the embedding: pp = cp = 1"
                self.mtp = nn.Module()
                self.mtp.layers = nn.ModuleList(
                    [MTPBlock(cfg, ps_, self.dtype, device, gen, k) for k in range(cfg.mtp_num_layers)])

        for n, p in self.named_parameters():
            if any(k in n for k in ("layernorm", "layer_norm", "router", "value_head", "shared_expert")) or n.endswith(".bias") and "linear_proj" in n:
                p.tp_replicated = True
        if hasattr(self, "embedding") and not self.pre_process:
            # the last stage's copy of an embedding the first stage owns (tied output layer, MTP blocks)
            self.embedding.word_embeddings.weight.pp_duplicate = True

    # ------------------------------------------------------------------ helpers
    def lm_head_weight(self):
        if self.cfg.tie_word_embeddings:
            return self.embedding.word_embeddings.weight
        return self.output_layer.weight

    def rope_tables(self, positions):
        return ops.rope_cos_sin(positions, self.cfg.rotary_dim, self.cfg.rope_theta, self.cfg.mrope_section)

    # ------------------------------------------------------------------ forward
    def forward(self, tokens=None, positions=None, cu_seqlens=None, hidden_in=None, attn_fn=None,
                inputs_embeds=None, max_seqlen=None, return_prenorm: bool = False):
        """tokens ``[T]`` (T divisible by tp when sequence-parallel).  Returns the
        normalised final hidden ``[T, H]`` on the last pipeline stage, else the
        stage output (sequence-parallel shard)."""
        sp = self.sequence_parallel
        if self.pre_process:
            h = inputs_embeds if inputs_embeds is not None else self.embedding.word_embeddings(tokens, sp)
            if inputs_embeds is not None and sp:
                h = TP.scatter_seq(h, self.ps.tp)
        else:
            h = hidden_in
        cos, sin = self.rope_tables(positions)
        if self.cfg.dsa_topk > 0 or self.cfg.multi_latent_attention:
            for layer in self.decoder.layers:
                layer.self_attention.positions = positions
        for layer in self.decoder.layers:
            if self.recompute and torch.is_grad_enabled():
                h = checkpoint(layer, h, cos, sin, cu_seqlens, attn_fn, max_seqlen, use_reentrant=False)
            else:
                h = layer(h, cos, sin, cu_seqlens, attn_fn, max_seqlen)
        if not self.post_process:
            return h
        prenorm = h
        h = ops.rmsnorm(h, self.decoder.final_layernorm.weight, self.cfg.rms_norm_eps)
        if sp:
            h = TP.gather_seq(h, self.ps.tp)
        if return_prenorm:   # the MTP blocks continue from the un-normalised stream (sequence-parallel shard)
            return h, prenorm
        return h

    def logits(self, hidden):
        """Local vocab shard of the logits (debug / rollout sampling)."""
        return ops.linear(hidden, self.lm_head_weight())

    def log_probs(self, hidden, targets, temperature: float = 1.0, with_entropy: bool = True):
        """Per-row log p(target) and entropy over the FULL vocabulary.
        Padded vocabulary rows (beyond ``cfg.vocab_size``) are excluded."""
        w = self.lm_head_weight()
        v_real = min(self.v_local, max(0, self.cfg.vocab_size - self.vocab_start))
        if v_real < self.v_local:
            w = w[:v_real]
        # sequence parallel: ``hidden`` came out of an all-gather whose backward is a
        # reduce-scatter, which already sums the partial (per vocab shard) gradients
        if not self.sequence_parallel:
            hidden = TP.copy_to_tp(hidden, self.ps.tp)
        return ops.fused_lm_head_logprob(hidden, w, targets, self.ps.tp.group, self.vocab_start, with_entropy, temperature)

    def class_logits(self, hidden):
        """Sequence-classification logits ``[rows, num_classes]`` from the given (last-token) hidden rows."""
        if self.sequence_parallel:
            hidden = _ScaleGrad.apply(hidden, 1.0 / self.ps.tp.size)
        return ops.linear(hidden, self.score.weight).float()

    def values(self, hidden):
        """Scalar value per row (critic).  The head is replicated over TP, so
        under sequence parallelism each rank's (identical) gradient is scaled by
        1/tp before the reduce-scatter sums them."""
        if self.sequence_parallel:
            hidden = _ScaleGrad.apply(hidden, 1.0 / self.ps.tp.size)
        return ops.linear(hidden, self.value_head.weight)[:, 0].float()


class _ScaleGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, s):
        ctx.s = s
        return x

    @staticmethod
    def backward(ctx, g):
        return g * ctx.s, None
