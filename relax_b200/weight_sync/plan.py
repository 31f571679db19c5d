"""Copy plan for trainer -> rollout weight synchronisation.

The trainer holds Megatron-layout shards (per-group interleaved QKV, ``[gate;
up]`` per TP shard, TP/PP/EP sharding of the trainer); the rollout engine holds
serving-layout shards (``[q | k | v]``, its own TP/EP).  Instead of gathering
full tensors, converting names/shapes and broadcasting them (the reference's
path: relax/backends/megatron/weight_update/common.py:20-126,
weight_conversion/qwen2.py, update_weight_from_distributed.py:351-376), this
module computes, once, a table of 2-D block copies

    (src rank, src tensor, row0, col0)  ->  (dst rank, dst tensor, row0, col0), rows x cols

that moves every element exactly once from a trainer shard straight into the
rollout parameter buffer.  The table is consumed by the CUDA weight-sync kernel
(peer stores over NVLink, optional cast/quantise) and by the CPU executor in
:mod:`relax_b200.weight_sync.sync`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable

from ..models.config import ModelConfig


@dataclass(frozen=True)
class BlockCopy:
    src_rank: int      # trainer-local rank index (tp + tp_size * (ep...)) see TrainerLayout.rank_of
    src_name: str      # trainer parameter name
    src_row: int
    src_col: int
    dst_rank: int      # rollout-engine-local rank (tp rank or ep rank)
    dst_name: str      # rollout parameter name
    dst_row: int
    dst_col: int
    rows: int
    cols: int
    src_batch: int = 0   # leading index for stacked expert tensors
    dst_batch: int = 0
    src_stage: int = 0   # pipeline stage of the trainer that owns the source tensor


@dataclass(frozen=True)
class TrainerLayout:
    tp: int = 1
    pp: int = 1
    ep: int = 1

    def layer_owner_pp(self, cfg: ModelConfig, layer: int) -> int:
        return layer // (cfg.num_layers // self.pp)


def _intersect(a0, a1, b0, b1):
    lo, hi = max(a0, b0), min(a1, b1)
    return (lo, hi) if lo < hi else None


def _row_sharded(canon_rows: int, src_parts: int, dst_parts: int):
    """Yield (src_part, src_off, dst_part, dst_off, n) for a dimension split evenly both ways."""
    s, d = canon_rows // src_parts, canon_rows // dst_parts
    for sp in range(src_parts):
        for dp in range(dst_parts):
            it = _intersect(sp * s, (sp + 1) * s, dp * d, (dp + 1) * d)
            if it:
                yield sp, it[0] - sp * s, dp, it[0] - dp * d, it[1] - it[0]


def _trainer_param_name(layer_local: int, kind: str) -> str:
    base = f"decoder.layers.{layer_local}."
    return {
        "qkv": base + "self_attention.linear_qkv.weight",
        "qkv_bias": base + "self_attention.linear_qkv.bias",
        "input_norm": base + "self_attention.linear_qkv.layer_norm_weight",
        "q_norm": base + "self_attention.q_layernorm.weight",
        "k_norm": base + "self_attention.k_layernorm.weight",
        "o": base + "self_attention.linear_proj.weight",
        "post_norm": base + "mlp.linear_fc1.layer_norm_weight",
        "post_norm_moe": base + "pre_mlp_layernorm.weight",
        "fc1": base + "mlp.linear_fc1.weight",
        "fc2": base + "mlp.linear_fc2.weight",
        "router": base + "mlp.router.weight",
        "experts_fc1": base + "mlp.experts.linear_fc1.weight",
        "experts_fc2": base + "mlp.experts.linear_fc2.weight",
        "router_bias": base + "mlp.router.expert_bias",
        "shared_fc1": base + "mlp.shared_experts.linear_fc1.weight",
        "shared_fc2": base + "mlp.shared_experts.linear_fc2.weight",
        "shared_gate": base + "mlp.shared_experts.gate_weight",
        "post_attn_norm": base + "post_self_attn_layernorm.weight",
        "post_mlp_norm": base + "post_mlp_layernorm.weight",
    }[kind]


trainer_param_name = _trainer_param_name


MTP_TRAINER_PREFIX = "mtp.layers.0."


def build_plan(cfg: ModelConfig, src: TrainerLayout, dst_tp: int, dst_ep: int = 1, mtp: bool = False) -> list[BlockCopy]:
    """All block copies for one rollout engine, sourced from ONE trainer
    data-parallel replica.  ``src_rank`` is the trainer TP rank for dense
    tensors and the EP rank for expert tensors (``src_batch`` = local expert);
    the pipeline stage that owns a layer is implied by the layer index.

    ``mtp``: also the first multi-token-prediction block (the engine's draft model for speculative decoding): its
    transformer layer becomes rollout layer ``num_layers``, its norms and projection ``mtp.*``; it lives on the last
    pipeline stage."""
    H, hd = cfg.hidden_size, cfg.head_dim
    ng, qpg = cfg.num_query_groups, cfg.num_attention_heads // cfg.num_query_groups
    plan: list[BlockCopy] = []
    per_stage = cfg.num_layers // src.pp
    add = plan.append

    def rep(src_name, dst_name, n):
        for r in range(dst_tp):
            add(BlockCopy(r % src.tp, src_name, 0, 0, r, dst_name, 0, 0, 1, n))

    # vocabulary-sharded tensors
    v_src = (cfg.vocab_size + src.tp - 1) // src.tp * src.tp
    v_dst = (cfg.vocab_size + dst_tp - 1) // dst_tp * dst_tp
    names = [("embedding.word_embeddings.weight", "embed")]
    if not cfg.tie_word_embeddings:
        names.append(("output_layer.weight", "lm_head"))
    for sname, dname in names:
        s, d = v_src // src.tp, v_dst // dst_tp
        for sp in range(src.tp):
            for dp in range(dst_tp):
                it = _intersect(sp * s, min((sp + 1) * s, cfg.vocab_size), dp * d, min((dp + 1) * d, cfg.vocab_size))
                if it:
                    add(BlockCopy(sp, sname, it[0] - sp * s, 0, dp, dname, it[0] - dp * d, 0, it[1] - it[0], H))
    rep("decoder.final_layernorm.weight", "final_norm", H)

    ng_s, ng_d = ng // src.tp, ng // dst_tp
    grp_rows = (qpg + 2) * hd
    layers = [(layer, layer % per_stage, None) for layer in range(cfg.num_layers)]
    if mtp:
        if cfg.mtp_num_layers < 1:
            raise ValueError("the model has no multi-token-prediction block to draft with")
        layers.append((cfg.num_layers, 0, MTP_TRAINER_PREFIX + "transformer_layer."))
        rep(MTP_TRAINER_PREFIX + "enorm.weight", "mtp.enorm", H)
        rep(MTP_TRAINER_PREFIX + "hnorm.weight", "mtp.hnorm", H)
        rep(MTP_TRAINER_PREFIX + "final_layernorm.weight", "mtp.final_norm", H)
        for r in range(dst_tp):
            add(BlockCopy(r % src.tp, MTP_TRAINER_PREFIX + "eh_proj.weight", 0, 0, r, "mtp.eh_proj", 0, 0, H, 2 * H))
    for layer, ll, base in layers:
        p = f"layers.{layer}."
        if base is not None:
            trainer_param_name = lambda l_, kind, _b=base: _trainer_param_name(l_, kind).replace("decoder.layers.0.", _b)  # noqa: E731
        else:
            trainer_param_name = _trainer_param_name
        rep(trainer_param_name(ll, "input_norm"), p + "input_norm", H)
        from ..models.hybrid import mixer_kind

        gdn_layer = mixer_kind(cfg, layer) == "gdn"
        if gdn_layer:
            # Gated DeltaNet mixer: whole tensors (hybrid stacks run with tp = 1 on both sides)
            if src.tp > 1 or dst_tp > 1:
                raise NotImplementedError("Gated-DeltaNet layers are synchronised between tp = 1 layouts")
            hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
            kd, vd = hk * d, hv * d
            gbase = trainer_param_name(ll, "o").replace("linear_proj.weight", "gdn.")
            for sname, dname, r_, c_ in (("in_proj_qkvz.weight", "gdn_qkvz", 2 * kd + 2 * vd, H), ("in_proj_ba.weight", "gdn_ba", 2 * hv, H),
                                        ("conv1d.weight", "gdn_conv", 2 * kd + vd, 4), ("out_proj.weight", "gdn_out", H, vd)):
                add(BlockCopy(0, gbase + sname, 0, 0, 0, p + dname, 0, 0, r_, c_))
            rep(gbase + "dt_bias", p + "gdn_dt_bias", hv)
            rep(gbase + "A_log", p + "gdn_A_log", hv)
            rep(gbase + "norm.weight", p + "gdn_norm", d)
        mla_layer = mixer_kind(cfg, layer) == "dsa"
        if mla_layer:
            if src.tp > 1 or dst_tp > 1:
                raise NotImplementedError("latent-attention layers are synchronised between tp = 1 layouts")
            nh, nope, rope, kvl, vh = cfg.num_attention_heads, cfg.dsa_nope, cfg.dsa_rope, cfg.dsa_kv_lora, cfg.dsa_v_head
            dbase = trainer_param_name(ll, "o").replace("linear_proj.weight", "dsa.")
            mats = [("linear_q_down_proj.weight", "mla_q_down", cfg.dsa_q_lora, H), ("linear_q_up_proj.weight", "mla_q_up", nh * (nope + rope), cfg.dsa_q_lora),
                    ("linear_kv_down_proj.weight", "mla_kv_down", kvl + rope, H), ("linear_kv_up_proj.weight", "mla_kv_up", nh * (nope + vh), kvl),
                    ("linear_proj.weight", "mla_o", H, nh * vh)]
            if cfg.dsa_topk > 0:
                mats += [("indexer.linear_wq.weight", "idx_wq", cfg.dsa_index_heads * cfg.dsa_index_dim, H),
                         ("indexer.linear_wk.weight", "idx_wk", cfg.dsa_index_dim, H), ("indexer.linear_weights.weight", "idx_w", cfg.dsa_index_heads, H)]
            for sname, dname, r_, c_ in mats:
                add(BlockCopy(0, dbase + sname, 0, 0, 0, p + dname, 0, 0, r_, c_))
            rep(dbase + "linear_q_up_proj.layer_norm_weight", p + "mla_q_norm", cfg.dsa_q_lora)
            rep(dbase + "linear_kv_up_proj.layer_norm_weight", p + "mla_kv_norm", kvl)
            gdn_layer = True            # from here on: no softmax-attention tensors for this layer
        if cfg.sandwich_norm:
            rep(trainer_param_name(ll, "post_attn_norm"), p + "post_attn_norm", H)
            rep(trainer_param_name(ll, "post_mlp_norm"), p + "post_mlp_norm", H)
        if cfg.qk_layernorm and not gdn_layer:
            rep(trainer_param_name(ll, "q_norm"), p + "q_norm", hd)
            rep(trainer_param_name(ll, "k_norm"), p + "k_norm", hd)
        # QKV: per global group g, three row blocks (with gated attention the group also holds one gate row per query
        # feature, between its query heads and its key: they go to a tensor of their own)
        nq_d, nkv_d = cfg.num_attention_heads // dst_tp, ng_d
        gate_rows = qpg * hd if cfg.attention_output_gate else 0
        for g in range(ng if not gdn_layer else 0):
            st, sg = g // ng_s, g % ng_s
            dt, dg = g // ng_d, g % ng_d
            sbase = sg * (grp_rows + gate_rows)
            blocks = (
                (sbase, dg * qpg * hd, qpg * hd),                      # q heads of the group
                (sbase + gate_rows + qpg * hd, nq_d * hd + dg * hd, hd),           # k
                (sbase + gate_rows + (qpg + 1) * hd, (nq_d + nkv_d) * hd + dg * hd, hd),  # v
            )
            for srow, drow, n in blocks:
                add(BlockCopy(st, trainer_param_name(ll, "qkv"), srow, 0, dt, p + "qkv", drow, 0, n, H))
                if cfg.qkv_bias:
                    add(BlockCopy(st, trainer_param_name(ll, "qkv_bias"), 0, srow, dt, p + "qkv_bias", 0, drow, 1, n))
            if gate_rows:
                add(BlockCopy(st, trainer_param_name(ll, "qkv"), sbase + qpg * hd, 0, dt, p + "attn_gate", dg * qpg * hd, 0, gate_rows, H))
        # o_proj: column sharded
        for sp, so, dp, do, n in (_row_sharded(cfg.q_size, src.tp, dst_tp) if not gdn_layer else ()):
            add(BlockCopy(sp, trainer_param_name(ll, "o"), 0, so, dp, p + "o", 0, do, H, n))
        is_moe = cfg.is_moe_layer(layer)
        if is_moe:
            rep(trainer_param_name(ll, "post_norm_moe"), p + "post_norm", H)
            for r in range(dst_tp):
                add(BlockCopy(r % src.tp, trainer_param_name(ll, "router"), 0, 0, r, p + "router", 0, 0, cfg.num_experts, H))
            if cfg.moe_router_bias:
                rep(trainer_param_name(ll, "router_bias"), p + "router_bias", cfg.num_experts)
            if cfg.moe_shared_expert_ffn > 0:      # replicated on both sides
                Fsh = cfg.moe_shared_expert_ffn
                for r in range(dst_tp):
                    add(BlockCopy(r % src.tp, trainer_param_name(ll, "shared_fc1"), 0, 0, r, p + "shared_gate_up", 0, 0, 2 * Fsh, H))
                    add(BlockCopy(r % src.tp, trainer_param_name(ll, "shared_fc2"), 0, 0, r, p + "shared_down", 0, 0, H, Fsh))
                if cfg.moe_shared_expert_gate:
                    rep(trainer_param_name(ll, "shared_gate"), p + "shared_gate", H)
            F = cfg.moe_ffn_hidden_size
            el_s, el_d = cfg.num_experts // src.ep, cfg.num_experts // dst_ep
            for e in range(cfg.num_experts):
                add(BlockCopy(e // el_s, trainer_param_name(ll, "experts_fc1"), 0, 0, e // el_d, p + "experts_gate_up",
                              0, 0, 2 * F, H, src_batch=e % el_s, dst_batch=e % el_d))
                add(BlockCopy(e // el_s, trainer_param_name(ll, "experts_fc2"), 0, 0, e // el_d, p + "experts_down",
                              0, 0, H, F, src_batch=e % el_s, dst_batch=e % el_d))
        else:
            rep(trainer_param_name(ll, "post_norm"), p + "post_norm", H)
            F = cfg.ffn_hidden_size
            Fs, Fd = F // src.tp, F // dst_tp
            for sp, so, dp, do, n in _row_sharded(F, src.tp, dst_tp):
                add(BlockCopy(sp, trainer_param_name(ll, "fc1"), so, 0, dp, p + "gate_up", do, 0, n, H))          # gate
                add(BlockCopy(sp, trainer_param_name(ll, "fc1"), Fs + so, 0, dp, p + "gate_up", Fd + do, 0, n, H))  # up
            for sp, so, dp, do, n in _row_sharded(F, src.tp, dst_tp):
                add(BlockCopy(sp, trainer_param_name(ll, "fc2"), 0, so, dp, p + "down", 0, do, H, n))
    if src.pp > 1:
        from dataclasses import replace as _replace

        def stage_of(b: BlockCopy) -> int:
            if b.dst_name.startswith("layers."):
                return min(int(b.dst_name.split(".")[1]) // per_stage, src.pp - 1)      # the MTP layer sits on the last stage
            if b.dst_name == "embed":
                return 0
            return src.pp - 1          # final norm, output layer
        plan = [_replace(b, src_stage=stage_of(b)) for b in plan]
    return plan


_ADAPTED = {"qkv": ("linear_qkv", True), "o": ("linear_proj", False), "gate_up": ("linear_fc1", True),
            "down": ("linear_fc2", False)}


def build_adapter_plan(cfg: ModelConfig, src: TrainerLayout, dst_tp: int, rank: int,
                       targets=("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2")) -> List[BlockCopy]:
    """Block copies that move LoRA factors instead of merged weights (adapter-mode sync,
    relax/backends/megatron/weight_update/lora_adapter_sync.py): derived from the weight plan, because the factor
    that is sharded follows its weight - ``B [out, r]`` of a column-parallel linear takes the weight's row blocks
    (including the grouped-QKV -> q | k | v and the [gate; up] re-layout), ``A [r, in]`` of a row-parallel linear its
    column blocks - while the other factor is replicated and copied whole to every rollout rank."""
    from dataclasses import replace as _replace

    H = cfg.hidden_size
    out, whole = [], set()
    for b in build_plan(cfg, src, dst_tp, 1):
        leaf = b.dst_name.rsplit(".", 1)[-1]
        if leaf not in _ADAPTED or not b.dst_name.startswith("layers.") or not b.src_name.endswith(".weight"):
            continue
        mod, column = _ADAPTED[leaf]
        if mod not in targets:
            continue
        base = b.src_name[: -len(".weight")]
        if column:
            out.append(_replace(b, src_name=base + ".lora_B", dst_name=b.dst_name + ".lora_B", src_col=0, dst_col=0, cols=rank))
            rep = (base + ".lora_A", b.dst_name + ".lora_A", rank, H)
        else:
            out.append(_replace(b, src_name=base + ".lora_A", dst_name=b.dst_name + ".lora_A", src_row=0, dst_row=0, rows=rank))
            rep = (base + ".lora_B", b.dst_name + ".lora_B", H, rank)
        if (rep[1], b.dst_rank) not in whole:
            whole.add((rep[1], b.dst_rank))
            out.append(BlockCopy(b.dst_rank % src.tp, rep[0], 0, 0, b.dst_rank, rep[1], 0, 0, rep[2], rep[3], src_stage=b.src_stage))
    return out


def plan_bytes(plan: Iterable[BlockCopy], itemsize: int = 2) -> int:
    return sum(b.rows * b.cols for b in plan) * itemsize
