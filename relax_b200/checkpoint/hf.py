"""Megatron-layout <-> Hugging Face name/shape conversion and safetensors IO.

Per family the reference keeps one converter (relax/backends/megatron/
weight_conversion/{qwen2,qwen3moe,llama,glm4,...}.py, dispatched by model name in
``__init__.py:24-93``): fused QKV is split by query group, ``linear_fc1`` is cut into
gate/up, norms fused into the following linear get their own HF names, experts are
numbered globally.  Here one table-driven converter covers the dense Qwen2/Qwen3/
Llama layouts and the Qwen3-MoE layout, in both directions, on FULL (unsharded)
tensors; sharded export gathers through :mod:`relax_b200.checkpoint.dist_ckpt`.
"""
from __future__ import annotations

import json
import os
import re
from typing import Iterable, Iterator, Optional

import torch

from ..models.config import ModelConfig

_LAYER = re.compile(r"decoder\.layers\.(\d+)\.(.+)")


def strip_prefix(name: str) -> str:
    while name.startswith("module."):
        name = name[len("module."):]
    return name


def _shared(cfg: ModelConfig) -> str:
    """HF module name of the shared expert: Qwen2-MoE / Qwen3-Next say ``shared_expert`` (and gate it), DeepSeek-V3 /
    GLM4-MoE say ``shared_experts``."""
    return "mlp.shared_expert" if cfg.moe_shared_expert_gate else "mlp.shared_experts"


def megatron_to_hf(cfg: ModelConfig, name: str, p: torch.Tensor) -> list:
    """One Megatron tensor -> list of ``(hf_name, tensor)``."""
    name = strip_prefix(name)
    H, hd = cfg.hidden_size, cfg.head_dim
    ng, qpg = cfg.num_query_groups, cfg.num_attention_heads // cfg.num_query_groups
    if name == "embedding.word_embeddings.weight":
        return [("model.embed_tokens.weight", p[: cfg.vocab_size])]
    if name == "output_layer.weight":
        return [("lm_head.weight", p[: cfg.vocab_size])]
    if name == "decoder.final_layernorm.weight":
        return [("model.norm.weight", p)]
    if name == "value_head.weight":
        return [("score.weight", p)]
    mt = re.match(r"mtp\.layers\.(\d+)\.(.+)", name)
    if mt and cfg.linear_attention_freq > 0:
        # Qwen3-Next / Qwen3.5 convention (relax/backends/megatron/weight_conversion/qwen3_next.py _convert_mtp_layer
        # :6-41): the block lives under ``mtp.*``; its projection takes [hidden | embedding], the other way round
        k_, sub = int(mt.group(1)), mt.group(2)
        own = {"enorm.weight": "mtp.pre_fc_norm_embedding.weight", "hnorm.weight": "mtp.pre_fc_norm_hidden.weight",
               "final_layernorm.weight": "mtp.norm.weight"}
        if sub in own:
            return [(own[sub], p)]
        if sub == "eh_proj.weight":
            e, h_ = p.chunk(2, dim=1)
            return [("mtp.fc.weight", torch.cat([h_, e], 1))]
        if sub.startswith("transformer_layer."):
            li = cfg.num_layers + k_              # the index the block's layer was built with
            return [(n.replace(f"model.layers.{li}.", f"mtp.layers.{k_}."), t)
                    for n, t in megatron_to_hf(cfg, f"decoder.layers.{li}." + sub[len("transformer_layer."):], p)]
        raise ValueError(f"unknown MTP parameter {name!r}")
    if mt:      # DeepSeek-V3 convention: MTP depth k lives at layer index num_layers + k
        li, sub = cfg.num_layers + int(mt.group(1)), mt.group(2)
        own = {"enorm.weight": "enorm.weight", "hnorm.weight": "hnorm.weight", "eh_proj.weight": "eh_proj.weight",
               "final_layernorm.weight": "shared_head.norm.weight"}
        if sub in own:
            return [(f"model.layers.{li}.{own[sub]}", p)]
        if sub.startswith("transformer_layer."):
            return megatron_to_hf(cfg, f"decoder.layers.{li}." + sub[len("transformer_layer."):], p)
        raise ValueError(f"unknown MTP parameter {name!r}")
    m = _LAYER.match(name)
    if not m:
        raise ValueError(f"unknown parameter name {name!r}")
    i, rest = m.groups()
    pre = f"model.layers.{i}."
    if rest == "self_attention.linear_qkv.weight":
        if cfg.attention_output_gate:
            # Qwen3.5 (HF Qwen3Next attention): q_proj holds, per head, the query rows followed by the gate rows
            x = p.view(ng, 2 * qpg + 2, hd, H)
            qg = torch.stack([x[:, :qpg], x[:, qpg:2 * qpg]], 2)          # [ng, qpg, 2, hd, H]
            return [(pre + "self_attn.q_proj.weight", qg.reshape(-1, H)),
                    (pre + "self_attn.k_proj.weight", x[:, 2 * qpg].reshape(-1, H)),
                    (pre + "self_attn.v_proj.weight", x[:, 2 * qpg + 1].reshape(-1, H))]
        x = p.view(ng, qpg + 2, hd, H)
        return [(pre + "self_attn.q_proj.weight", x[:, :qpg].reshape(-1, H)),
                (pre + "self_attn.k_proj.weight", x[:, qpg].reshape(-1, H)),
                (pre + "self_attn.v_proj.weight", x[:, qpg + 1].reshape(-1, H))]
    if rest == "self_attention.linear_qkv.bias":
        x = p.view(ng, qpg + 2, hd)
        return [(pre + "self_attn.q_proj.bias", x[:, :qpg].reshape(-1)), (pre + "self_attn.k_proj.bias", x[:, qpg].reshape(-1)),
                (pre + "self_attn.v_proj.bias", x[:, qpg + 1].reshape(-1))]
    if rest.startswith("self_attention.gdn."):
        return _gdn_to_hf(cfg, pre, rest[len("self_attention.gdn."):], p)
    if rest.startswith("self_attention.dsa."):
        sub = rest[len("self_attention.dsa."):]
        if sub not in _MLA_NAMES:
            raise ValueError(f"unknown latent-attention parameter {rest!r}")
        return [(pre + "self_attn." + _MLA_NAMES[sub], p)]
    simple = {
        "self_attention.linear_proj.weight": "self_attn.o_proj.weight",
        "self_attention.linear_qkv.layer_norm_weight": "input_layernorm.weight",
        "self_attention.q_layernorm.weight": "self_attn.q_norm.weight",
        "self_attention.k_layernorm.weight": "self_attn.k_norm.weight",
        "mlp.linear_fc1.layer_norm_weight": "post_attention_layernorm.weight",
        "pre_mlp_layernorm.weight": "post_attention_layernorm.weight",
        "mlp.linear_fc2.weight": "mlp.down_proj.weight",
        "post_self_attn_layernorm.weight": "post_self_attn_layernorm.weight",      # GLM-4 sandwich norms
        "post_mlp_layernorm.weight": "post_mlp_layernorm.weight",
        "mlp.router.weight": "mlp.gate.weight",
        "mlp.router.expert_bias": "mlp.gate.e_score_correction_bias",
        "mlp.shared_experts.linear_fc2.weight": _shared(cfg) + ".down_proj.weight",
        "mlp.shared_experts.gate_weight": "mlp.shared_expert_gate.weight",
    }
    if rest in simple:
        return [(pre + simple[rest], p)]
    if rest == "mlp.shared_experts.linear_fc1.weight":
        g, u = p.chunk(2, 0)
        return [(pre + _shared(cfg) + ".gate_proj.weight", g), (pre + _shared(cfg) + ".up_proj.weight", u)]
    if rest == "mlp.linear_fc1.weight":
        g, u = p.chunk(2, 0)
        return [(pre + "mlp.gate_proj.weight", g), (pre + "mlp.up_proj.weight", u)]
    if rest == "mlp.experts.linear_fc1.weight":      # stacked [E, 2F, H]
        out = []
        for e in range(p.shape[0]):
            g, u = p[e].chunk(2, 0)
            out += [(pre + f"mlp.experts.{e}.gate_proj.weight", g), (pre + f"mlp.experts.{e}.up_proj.weight", u)]
        return out
    if rest == "mlp.experts.linear_fc2.weight":
        return [(pre + f"mlp.experts.{e}.down_proj.weight", p[e]) for e in range(p.shape[0])]
    raise ValueError(f"unknown layer parameter {rest!r}")


# multi-head latent attention under its DeepSeek-V3 names (relax/backends/megatron/weight_conversion/deepseekv3.py); the
# lightning indexer of the sparse variant keeps its own small projections next to them
_MLA_NAMES = {
    "linear_q_down_proj.weight": "q_a_proj.weight", "linear_q_up_proj.layer_norm_weight": "q_a_layernorm.weight",
    "linear_q_up_proj.weight": "q_b_proj.weight", "linear_kv_down_proj.weight": "kv_a_proj_with_mqa.weight",
    "linear_kv_up_proj.layer_norm_weight": "kv_a_layernorm.weight", "linear_kv_up_proj.weight": "kv_b_proj.weight",
    "linear_proj.weight": "o_proj.weight", "indexer.linear_wq.weight": "indexer.wq_b.weight",
    "indexer.linear_wk.weight": "indexer.wk.weight", "indexer.linear_weights.weight": "indexer.weights_proj.weight",
}


def _gdn_perm(cfg: ModelConfig, what: str) -> torch.Tensor:
    """Row order that turns this package's flat Gated-DeltaNet projections into the Hugging Face ones.  Here the rows
    of ``in_proj_qkvz`` are ``[q of all key heads | k | v of all value heads | z]`` and those of ``in_proj_ba``
    ``[b | a]``; Hugging Face (Qwen3-Next ``fix_query_key_value_ordering``) groups them per KEY head:
    ``[q_h | k_h | v of the head's value heads | z of the same]`` and ``[b of the head's value heads | a ...]``."""
    hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
    r, kd, vd = hv // hk, hk * d, hv * d
    rows = []
    for h in range(hk):
        if what == "qkvz":
            rows += list(range(h * d, (h + 1) * d))                                  # q_h
            rows += list(range(kd + h * d, kd + (h + 1) * d))                        # k_h
            rows += list(range(2 * kd + h * r * d, 2 * kd + (h + 1) * r * d))        # v of value heads h*r .. h*r + r - 1
            rows += list(range(2 * kd + vd + h * r * d, 2 * kd + vd + (h + 1) * r * d))   # z of the same heads
        else:
            rows += list(range(h * r, (h + 1) * r)) + list(range(hv + h * r, hv + (h + 1) * r))
    return torch.tensor(rows)


def _gdn_to_hf(cfg: ModelConfig, pre: str, sub: str, p: torch.Tensor) -> list:
    """Gated-DeltaNet tensors under their Qwen3-Next names (relax/backends/megatron/weight_conversion/qwen3_next.py
    :176-184 passes ``linear_attn.*`` through)."""
    la = pre + "linear_attn."
    if sub == "in_proj_qkvz.weight":
        return [(la + sub, p.index_select(0, _gdn_perm(cfg, "qkvz").to(p.device)))]
    if sub == "in_proj_ba.weight":
        return [(la + sub, p.index_select(0, _gdn_perm(cfg, "ba").to(p.device)))]
    if sub == "conv1d.weight":
        return [(la + sub, p.unsqueeze(1))]              # [channels, 1, taps]: channels are [q | k | v] on both sides
    if sub in ("dt_bias", "A_log", "norm.weight", "out_proj.weight"):
        return [(la + sub, p)]
    raise ValueError(f"unknown Gated-DeltaNet parameter {sub!r}")


def _gdn_from_hf(cfg: ModelConfig, hf: dict, pre: str, b: str, out: dict) -> None:
    la, g = pre + "linear_attn.", b + "self_attention.gdn."
    for what in ("qkvz", "ba"):
        perm = _gdn_perm(cfg, what)
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(perm.numel())
        w = hf[la + f"in_proj_{what}.weight"]
        out[g + f"in_proj_{what}.weight"] = w.index_select(0, inv.to(w.device))
    c = hf[la + "conv1d.weight"]
    out[g + "conv1d.weight"] = c[:, 0] if c.dim() == 3 else c
    for sub in ("dt_bias", "A_log", "norm.weight", "out_proj.weight"):
        out[g + sub] = hf[la + sub]


_NORM_SUFFIXES = ("norm.weight", "layernorm.weight", "layer_norm_weight")


def _is_norm(name: str) -> bool:
    """Norm weights that a zero-centred checkpoint stores as ``gamma - 1``.  The gated norm inside a Gated-DeltaNet
    mixer is an ordinary RMSNorm in those checkpoints too (Qwen3-Next ``Qwen3NextRMSNormGated``)."""
    return name.endswith(_NORM_SUFFIXES) and "linear_attn.norm." not in name


def _vision_to_hf(cfg: ModelConfig, name: str, t: torch.Tensor) -> list:
    """One tensor of the vision tower (``vision.*`` in the trainer's state) under its Qwen2.5-VL checkpoint name(s)."""
    v = cfg.vision
    f = v.ffn_hidden_size
    fp = (f + 63) // 64 * 64
    n = name[len("vision."):]
    pre = "model.visual."
    top = {"patch_embed": ("patch_embed.proj.weight", lambda x: x.reshape(v.hidden_size, v.in_channels, v.temporal_patch_size, v.patch_size, v.patch_size)),
           "merger_norm": ("merger.ln_q.weight", None), "merger_fc1": ("merger.mlp.0.weight", None), "merger_fc1_bias": ("merger.mlp.0.bias", None),
           "merger_fc2": ("merger.mlp.2.weight", None), "merger_fc2_bias": ("merger.mlp.2.bias", None)}
    if n in top:
        hk, fn = top[n]
        return [(pre + hk, fn(t) if fn else t)]
    m = re.match(r"blocks\.(\d+)\.(\w+)$", n)
    if not m:
        raise ValueError(f"unknown vision tower parameter {name!r}")
    b, leaf = pre + f"blocks.{m.group(1)}.", m.group(2)
    simple = {"norm1": "norm1.weight", "norm2": "norm2.weight", "qkv": "attn.qkv.weight", "qkv_bias": "attn.qkv.bias",
              "proj": "attn.proj.weight", "proj_bias": "attn.proj.bias", "fc2_bias": "mlp.down_proj.bias"}
    if leaf in simple:
        return [(b + simple[leaf], t)]
    if leaf == "fc1":
        return [(b + "mlp.gate_proj.weight", t[:f]), (b + "mlp.up_proj.weight", t[fp:fp + f])]
    if leaf == "fc1_bias":
        return [(b + "mlp.gate_proj.bias", t[:f]), (b + "mlp.up_proj.bias", t[fp:fp + f])]
    if leaf == "fc2":
        return [(b + "mlp.down_proj.weight", t[:, :f])]
    raise ValueError(f"unknown vision tower parameter {name!r}")


def convert_state_to_hf(cfg: ModelConfig, state: dict) -> dict:
    out = {}
    vl = cfg.vision is not None and any(strip_prefix(k).startswith("vision.") for k in state)
    for k, v in state.items():
        if strip_prefix(k).startswith("vision."):
            for hk, hv in _vision_to_hf(cfg, strip_prefix(k), v):
                out[hk] = hv.contiguous()
            continue
        for hk, hv in megatron_to_hf(cfg, k, v):
            if vl and hk.startswith("model."):       # vision-language layout: the decoder lives under model.language_model.*
                hk = "model.language_model." + hk[len("model."):]
            # zero-centred norms (Qwen3.5, ``--apply-layernorm-1p``): the checkpoint stores gamma - 1, the model here
            # keeps gamma itself, so the offset lives in the conversion only
            out[hk] = (hv - 1.0).contiguous() if (cfg.layernorm_zero_centered and _is_norm(hk)) else hv.contiguous()
    if cfg.tie_word_embeddings:
        out.pop("lm_head.weight", None)
    return out


def hf_to_megatron_state(cfg: ModelConfig, hf: dict) -> dict:
    """Full HF state dict -> full Megatron-layout state dict (inverse of :func:`convert_state_to_hf`)."""
    if cfg.layernorm_zero_centered:
        hf = {k: (v + 1.0 if _is_norm(k) else v) for k, v in hf.items()}
    H, hd = cfg.hidden_size, cfg.head_dim
    ng, qpg = cfg.num_query_groups, cfg.num_attention_heads // cfg.num_query_groups
    out = {"embedding.word_embeddings.weight": hf["model.embed_tokens.weight"],
           "decoder.final_layernorm.weight": hf["model.norm.weight"]}
    if not cfg.tie_word_embeddings:
        out["output_layer.weight"] = hf.get("lm_head.weight", hf["model.embed_tokens.weight"])
    for i in range(cfg.num_layers + cfg.mtp_num_layers):
        pre, b = f"model.layers.{i}.", f"decoder.layers.{i}."
        if i >= cfg.num_layers and cfg.linear_attention_freq > 0:        # Qwen3-Next style ``mtp.*`` names
            k = i - cfg.num_layers
            pre, b = f"mtp.layers.{k}.", f"mtp.layers.{k}.transformer_layer."
            out[f"mtp.layers.{k}.enorm.weight"] = hf["mtp.pre_fc_norm_embedding.weight"]
            out[f"mtp.layers.{k}.hnorm.weight"] = hf["mtp.pre_fc_norm_hidden.weight"]
            out[f"mtp.layers.{k}.final_layernorm.weight"] = hf["mtp.norm.weight"]
            h_, e = hf["mtp.fc.weight"].chunk(2, dim=1)
            out[f"mtp.layers.{k}.eh_proj.weight"] = torch.cat([e, h_], 1)
        elif i >= cfg.num_layers:
            k = i - cfg.num_layers
            b = f"mtp.layers.{k}.transformer_layer."
            out[f"mtp.layers.{k}.enorm.weight"] = hf[pre + "enorm.weight"]
            out[f"mtp.layers.{k}.hnorm.weight"] = hf[pre + "hnorm.weight"]
            out[f"mtp.layers.{k}.eh_proj.weight"] = hf[pre + "eh_proj.weight"]
            out[f"mtp.layers.{k}.final_layernorm.weight"] = hf[pre + "shared_head.norm.weight"]
        from ..models.hybrid import mixer_kind

        kind = mixer_kind(cfg, i)          # the draft block's layer is built by the same rule, from its index
        if kind == "gdn":
            _gdn_from_hf(cfg, hf, pre, b, out)
        elif kind == "dsa":
            for ours, theirs in _MLA_NAMES.items():
                if (pre + "self_attn." + theirs) in hf:
                    out[b + "self_attention.dsa." + ours] = hf[pre + "self_attn." + theirs]
        if kind != "attention":
            out[b + "self_attention.linear_qkv.layer_norm_weight"] = hf[pre + "input_layernorm.weight"]
            _mlp_from_hf(cfg, hf, i, pre, b, out)
            continue
        k = hf[pre + "self_attn.k_proj.weight"].view(ng, 1, hd, H)
        v = hf[pre + "self_attn.v_proj.weight"].view(ng, 1, hd, H)
        if cfg.attention_output_gate:
            qg = hf[pre + "self_attn.q_proj.weight"].view(ng, qpg, 2, hd, H)
            out[b + "self_attention.linear_qkv.weight"] = torch.cat([qg[:, :, 0], qg[:, :, 1], k, v], 1).reshape(-1, H)
        else:
            q = hf[pre + "self_attn.q_proj.weight"].view(ng, qpg, hd, H)
            out[b + "self_attention.linear_qkv.weight"] = torch.cat([q, k, v], 1).reshape(-1, H)
        if cfg.qkv_bias:
            qb = hf[pre + "self_attn.q_proj.bias"].view(ng, qpg, hd)
            kb = hf[pre + "self_attn.k_proj.bias"].view(ng, 1, hd)
            vb = hf[pre + "self_attn.v_proj.bias"].view(ng, 1, hd)
            out[b + "self_attention.linear_qkv.bias"] = torch.cat([qb, kb, vb], 1).reshape(-1)
        out[b + "self_attention.linear_proj.weight"] = hf[pre + "self_attn.o_proj.weight"]
        out[b + "self_attention.linear_qkv.layer_norm_weight"] = hf[pre + "input_layernorm.weight"]
        if cfg.sandwich_norm:
            out[b + "post_self_attn_layernorm.weight"] = hf[pre + "post_self_attn_layernorm.weight"]
            out[b + "post_mlp_layernorm.weight"] = hf[pre + "post_mlp_layernorm.weight"]
        if cfg.qk_layernorm:
            out[b + "self_attention.q_layernorm.weight"] = hf[pre + "self_attn.q_norm.weight"]
            out[b + "self_attention.k_layernorm.weight"] = hf[pre + "self_attn.k_norm.weight"]
        _mlp_from_hf(cfg, hf, i, pre, b, out)
    return out


def _mlp_from_hf(cfg: ModelConfig, hf: dict, i: int, pre: str, b: str, out: dict) -> None:
    """The feed-forward half of layer ``i`` (dense or mixture of experts) and the norm in front of it."""
    if True:
        if cfg.is_moe_layer(i):
            out[b + "pre_mlp_layernorm.weight"] = hf[pre + "post_attention_layernorm.weight"]
            out[b + "mlp.router.weight"] = hf[pre + "mlp.gate.weight"]
            if cfg.moe_router_bias:
                out[b + "mlp.router.expert_bias"] = hf[pre + "mlp.gate.e_score_correction_bias"]
            if cfg.moe_shared_expert_ffn > 0:
                sh = pre + _shared(cfg)
                out[b + "mlp.shared_experts.linear_fc1.weight"] = torch.cat([hf[sh + ".gate_proj.weight"], hf[sh + ".up_proj.weight"]], 0)
                out[b + "mlp.shared_experts.linear_fc2.weight"] = hf[sh + ".down_proj.weight"]
                if cfg.moe_shared_expert_gate:
                    out[b + "mlp.shared_experts.gate_weight"] = hf[pre + "mlp.shared_expert_gate.weight"]
            out[b + "mlp.experts.linear_fc1.weight"] = torch.stack(
                [torch.cat([hf[pre + f"mlp.experts.{e}.gate_proj.weight"], hf[pre + f"mlp.experts.{e}.up_proj.weight"]], 0)
                 for e in range(cfg.num_experts)])
            out[b + "mlp.experts.linear_fc2.weight"] = torch.stack(
                [hf[pre + f"mlp.experts.{e}.down_proj.weight"] for e in range(cfg.num_experts)])
        else:
            out[b + "mlp.linear_fc1.layer_norm_weight"] = hf[pre + "post_attention_layernorm.weight"]
            out[b + "mlp.linear_fc1.weight"] = torch.cat([hf[pre + "mlp.gate_proj.weight"], hf[pre + "mlp.up_proj.weight"]], 0)
            out[b + "mlp.linear_fc2.weight"] = hf[pre + "mlp.down_proj.weight"]


def hf_config_dict(cfg: ModelConfig) -> dict:
    arch = "DeepseekV3ForCausalLM" if (cfg.is_moe and cfg.moe_router_score == "sigmoid") else "Qwen3MoeForCausalLM" if cfg.is_moe else ("Qwen3ForCausalLM" if cfg.qk_layernorm else "Qwen2ForCausalLM")
    d = {"architectures": [arch], "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
         "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_query_groups,
         "head_dim": cfg.head_dim, "intermediate_size": cfg.ffn_hidden_size, "vocab_size": cfg.vocab_size,
         "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta, "tie_word_embeddings": cfg.tie_word_embeddings,
         "torch_dtype": "bfloat16", "hidden_act": "silu"}
    if cfg.is_moe:
        d.update(num_experts=cfg.num_experts, num_experts_per_tok=cfg.moe_top_k, moe_intermediate_size=cfg.moe_ffn_hidden_size,
                 norm_topk_prob=cfg.moe_router_norm_topk_prob)
        if cfg.moe_shared_expert_ffn > 0:
            d.update(n_shared_experts=1, shared_expert_intermediate_size=cfg.moe_shared_expert_ffn)
        if cfg.moe_first_dense_layers:
            d.update(first_k_dense_replace=cfg.moe_first_dense_layers)
        if cfg.moe_router_score == "sigmoid":
            d.update(scoring_func="sigmoid", routed_scaling_factor=cfg.moe_routed_scaling_factor, n_routed_experts=cfg.num_experts)
        if cfg.moe_router_bias:         # aux-loss-free balancing: a selection bias per expert (DeepSeek-V3 "noaux_tc")
            d["topk_method"] = "noaux_tc"
    d["attention_bias"] = bool(cfg.qkv_bias)
    if not cfg.is_moe and not cfg.qk_layernorm and not cfg.qkv_bias:
        d["architectures"] = ["LlamaForCausalLM"]
    if cfg.rotary_percent < 1.0:
        d["partial_rotary_factor"] = cfg.rotary_percent
    if cfg.linear_attention_freq > 0:
        # Qwen3-Next / Qwen3.5: every ``full_attention_interval``-th layer is (gated) softmax attention, the others
        # Gated DeltaNet with these head counts; norms are stored zero-centred
        d.update(architectures=["Qwen3NextForCausalLM"], model_type="qwen3_next", full_attention_interval=cfg.linear_attention_freq,
                 linear_num_key_heads=cfg.gdn_k_heads, linear_num_value_heads=cfg.gdn_v_heads, linear_key_head_dim=cfg.gdn_head_dim,
                 linear_value_head_dim=cfg.gdn_head_dim, linear_conv_kernel_dim=4, attn_output_gate=bool(cfg.attention_output_gate),
                 zero_centered_norms=bool(cfg.layernorm_zero_centered))
    elif cfg.dsa_topk > 0 or cfg.multi_latent_attention:
        # DeepSeek-V3 / GLM-MoE-DSA: latent attention ranks and head splits; ``index_topk`` > 0 adds the lightning indexer
        d.update(architectures=["GlmMoeDsaForCausalLM" if cfg.dsa_topk > 0 else "DeepseekV3ForCausalLM"],
                 model_type="glm_moe_dsa" if cfg.dsa_topk > 0 else "deepseek_v3", q_lora_rank=cfg.dsa_q_lora, kv_lora_rank=cfg.dsa_kv_lora,
                 qk_nope_head_dim=cfg.dsa_nope, qk_rope_head_dim=cfg.dsa_rope, v_head_dim=cfg.dsa_v_head, index_topk=cfg.dsa_topk,
                 index_n_heads=cfg.dsa_index_heads, index_head_dim=cfg.dsa_index_dim)
    elif cfg.sandwich_norm:
        d.update(architectures=["Glm4ForCausalLM"], model_type="glm4")
    if cfg.layernorm_zero_centered:
        d["zero_centered_norms"] = True
    return d


# ----------------------------------------------------------------------------- safetensors, sharded by size


def save_hf_checkpoint(directory: str, cfg: ModelConfig, hf_state: dict, max_shard_bytes: int = 5 << 30,
                       quantize_fp8: bool = False, fp8_block: int = 128, post_hook=None):
    """Write ``model-0000x-of-0000y.safetensors`` + index + ``config.json``.  With
    ``quantize_fp8`` every 2-D projection weight is stored as e4m3 with a
    ``weight_scale_inv`` tensor (block ``fp8_block``), the layout of the reference's
    streaming fp8 writer (relax/backends/megatron/model.py:1609-1653)."""
    from safetensors.torch import save_file

    from .. import ops

    os.makedirs(directory, exist_ok=True)
    items = []
    for k, v in hf_state.items():
        v = v.detach()
        if quantize_fp8 and v.dim() == 2 and "proj" in k and k.endswith(".weight"):
            q, s = ops.blockwise_cast_to_fp8(v, fp8_block)
            items.append((k, q.cpu()))
            items.append((k + "_scale_inv", s.cpu()))
        else:
            items.append((k, v.cpu().contiguous()))
    shards, cur, cur_bytes = [], {}, 0
    for k, v in items:
        nb = v.numel() * v.element_size()
        if cur and cur_bytes + nb > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[k] = v
        cur_bytes += nb
    if cur:
        shards.append(cur)
    weight_map, total = {}, 0
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors" if len(shards) > 1 else "model.safetensors"
        save_file(sh, os.path.join(directory, fn), metadata={"format": "pt"})
        for k, v in sh.items():
            weight_map[k] = fn
            total += v.numel() * v.element_size()
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1)
    c = hf_config_dict(cfg)
    if quantize_fp8:
        c["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [fp8_block, fp8_block],
                                    "activation_scheme": "dynamic"}
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(c, f, indent=1)
    if post_hook is not None:
        post_hook(directory)


def load_hf_checkpoint(directory: str, dequantize: bool = True, dtype=None) -> dict:
    from safetensors import safe_open

    from .. import ops

    if "://" in directory:   # object-store or file:// source: mirrored once per node, then read locally
        from ..utils.model_source import resolve_model_path

        directory = resolve_model_path(directory, local_rank=int(os.environ.get("LOCAL_RANK", "0")))
    files = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {directory}")
    out = {}
    for fn in files:
        with safe_open(os.path.join(directory, fn), framework="pt") as f:
            for k in f.keys():
                out[k] = f.get_tensor(k)
    if dequantize:
        for k in [k for k in out if k.endswith("_scale_inv")]:
            base = k[: -len("_scale_inv")]
            s = out.pop(k)
            block = 128
            cfgp = os.path.join(directory, "config.json")
            if os.path.exists(cfgp):
                block = json.load(open(cfgp)).get("quantization_config", {}).get("weight_block_size", [128])[0]
            out[base] = ops.blockwise_dequant_fp8(out[base], s, block, dtype or torch.bfloat16)
    if dtype is not None:
        out = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in out.items()}
    return out


def is_hf_checkpoint(path: str) -> bool:
    return os.path.isdir(path) and os.path.exists(os.path.join(path, "config.json")) and \
        any(f.endswith(".safetensors") for f in os.listdir(path))


def load_hf_into_model(path: str, cfg: ModelConfig, ps, model, strict: bool = True) -> list:
    """Read a Hugging Face checkpoint (local directory, ``file://`` or ``s3://``), convert it to the Megatron layout
    and copy this rank's shards into ``model`` (``--hf-checkpoint`` / ``--ref-load`` of the reference,
    relax/backends/megatron/checkpoint.py _load_checkpoint_hf :250-278)."""
    from .dist_ckpt import load_full_state

    dtype = next(model.parameters()).dtype
    hf = load_hf_checkpoint(path, dequantize=True, dtype=dtype)
    if any(k.startswith("model.language_model.") for k in hf):
        # vision-language checkpoints keep the decoder under model.language_model.* (and the tower under model.visual.*)
        hf = {("model." + k[len("model.language_model."):] if k.startswith("model.language_model.") else k): v for k, v in hf.items()}
    tower = getattr(model, "vision", None)
    missing = []
    if tower is not None:
        from ..models.vision import load_vision_from_hf

        missing += load_vision_from_hf(tower, hf, strict=strict)
    lm = {k: v for k, v in hf.items() if not k.startswith(("visual.", "model.visual."))}
    full = hf_to_megatron_state(cfg, lm)
    if tower is not None:       # the tower's tensors were filled above: leave them out of the layout-aware load
        named = [(n, p) for n, p in model.named_parameters() if not n.startswith("vision.")]
        return missing + load_full_state(cfg, ps, _NamedView(named), full, strict)
    return load_full_state(cfg, ps, model, full, strict)


class _NamedView:
    """Just enough of a module for ``load_full_state``: a fixed list of named parameters."""

    def __init__(self, named):
        self._named = list(named)

    def named_parameters(self):
        return iter(self._named)

    def parameters(self):
        return (p for _, p in self._named)


def config_from_hf(path: str) -> ModelConfig:
    """``config.json`` of a Hugging Face checkpoint -> :class:`ModelConfig` (the inverse of :func:`hf_config_dict`;
    the reference cross-checks its Megatron flags against this file, relax/backends/megatron/arguments.py)."""
    import json

    with open(os.path.join(path, "config.json")) as f:
        d = json.load(f)
    arch = (d.get("architectures") or [""])[0]
    heads = d["num_attention_heads"]
    kw = dict(name=os.path.basename(os.path.normpath(path)) or "hf", num_layers=d["num_hidden_layers"], hidden_size=d["hidden_size"],
              num_attention_heads=heads, num_query_groups=d.get("num_key_value_heads", heads),
              head_dim=d.get("head_dim") or d["hidden_size"] // heads, ffn_hidden_size=d.get("intermediate_size", 4 * d["hidden_size"]),
              vocab_size=d["vocab_size"], rms_norm_eps=d.get("rms_norm_eps", 1e-6), rope_theta=float(d.get("rope_theta", 1e6)),
              tie_word_embeddings=bool(d.get("tie_word_embeddings", False)), qk_layernorm="Qwen3" in arch,
              qkv_bias="Qwen2" in arch)
    n_exp = d.get("num_experts") or d.get("n_routed_experts") or 0
    if n_exp:
        kw.update(num_experts=n_exp, moe_top_k=d.get("num_experts_per_tok", 8), moe_ffn_hidden_size=d.get("moe_intermediate_size", kw["ffn_hidden_size"]),
                  moe_router_norm_topk_prob=bool(d.get("norm_topk_prob", True)), moe_shared_expert_ffn=d.get("shared_expert_intermediate_size", 0) or 0,
                  moe_first_dense_layers=d.get("first_k_dense_replace", 0) or 0)
        if d.get("scoring_func") == "sigmoid":
            kw.update(moe_router_score="sigmoid", moe_routed_scaling_factor=float(d.get("routed_scaling_factor", 1.0)))
        if d.get("topk_method") == "noaux_tc":
            kw["moe_router_bias"] = True
    if "attention_bias" in d:
        kw["qkv_bias"] = bool(d["attention_bias"])
    if d.get("partial_rotary_factor") is not None:
        kw["rotary_percent"] = float(d["partial_rotary_factor"])
    if d.get("full_attention_interval"):            # Qwen3-Next / Qwen3.5 hybrids
        kw.update(linear_attention_freq=int(d["full_attention_interval"]), gdn_k_heads=d.get("linear_num_key_heads", 2),
                  gdn_v_heads=d.get("linear_num_value_heads", 4), gdn_head_dim=d.get("linear_key_head_dim", 32),
                  attention_output_gate=bool(d.get("attn_output_gate", True)), qk_layernorm=True,
                  layernorm_zero_centered=bool(d.get("zero_centered_norms", True)))
    elif d.get("kv_lora_rank"):                     # DeepSeek-V3 / GLM-MoE-DSA latent attention
        kw.update(dsa_q_lora=d.get("q_lora_rank") or 64, dsa_kv_lora=d["kv_lora_rank"], dsa_nope=d.get("qk_nope_head_dim", 16),
                  dsa_rope=d.get("qk_rope_head_dim", 8), dsa_v_head=d.get("v_head_dim", 16), dsa_topk=int(d.get("index_topk", 0) or 0),
                  dsa_index_heads=d.get("index_n_heads", 4), dsa_index_dim=d.get("index_head_dim", 16), qkv_bias=False)
        kw["multi_latent_attention"] = kw["dsa_topk"] == 0
    elif "Glm4" in arch:
        kw.update(sandwich_norm=True, qk_layernorm=False)
    if "zero_centered_norms" in d:
        kw["layernorm_zero_centered"] = bool(d["zero_centered_norms"])
    return ModelConfig(**kw)


def validate_against_hf(cfg: ModelConfig, path: str) -> None:
    """Stop when the model the flags / preset describe is not the model whose ``config.json`` sits under ``path``
    (relax/backends/megatron/arguments.py _hf_validate_args :209-263 compares the same fields): a mismatch would
    otherwise surface as a shape error in the middle of the load or, worse, as silently wrong rotary / norm constants."""
    if not os.path.isfile(os.path.join(path, "config.json")):
        return
    hf = config_from_hf(path)
    fields = ["hidden_size", "num_attention_heads", "num_query_groups", "num_layers", "head_dim", "vocab_size",
              "tie_word_embeddings", "rope_theta", "rms_norm_eps"]
    if cfg.is_moe or hf.is_moe:
        fields += ["num_experts", "moe_top_k", "moe_ffn_hidden_size", "moe_shared_expert_ffn"]
    if not cfg.is_moe or cfg.moe_first_dense_layers > 0:
        fields.append("ffn_hidden_size")
    errors = []
    for f in fields:
        a, b = getattr(cfg, f), getattr(hf, f)
        same = abs(float(a) - float(b)) <= 1e-12 * max(1.0, abs(float(b))) if isinstance(a, float) or isinstance(b, float) else a == b
        if not same:
            errors.append(f"{f}: {a} here, {b} in {os.path.join(path, 'config.json')}")
    if errors:
        raise ValueError("the model configuration does not match the Hugging Face checkpoint: " + "; ".join(errors))


def load_hf_into_rollout(path: str, cfg: ModelConfig, rollout_weights) -> None:
    """Fill a rollout engine's parameter buffer straight from a Hugging Face checkpoint (a grader or any serving-only
    model that has no trainer): HF names -> Megatron layout -> the block-copy plan the weight sync uses."""
    from ..weight_sync.plan import TrainerLayout, build_plan
    from ..weight_sync.sync import apply_block

    full = hf_to_megatron_state(cfg, load_hf_checkpoint(path, dequantize=True, dtype=rollout_weights.dtype))
    for b in build_plan(cfg, TrainerLayout(1, 1, 1), rollout_weights.tp_size, rollout_weights.ep_size,
                        mtp=bool(getattr(rollout_weights, "mtp", False))):         # the draft block too, when the engine speculates
        mine = rollout_weights.ep_rank if ".experts." in b.src_name else rollout_weights.tp_rank
        if b.dst_rank == mine:
            apply_block(b, full[b.src_name].to(rollout_weights.device), rollout_weights.p[b.dst_name])
