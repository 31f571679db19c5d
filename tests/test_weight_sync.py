"""The block-copy plan must reproduce gather -> convert -> shard bit-exactly."""
import pytest
import torch

from relax_b200.models.config import get_config
from relax_b200.models.transformer import GPTModel
from relax_b200.parallel.state import GroupInfo, ParallelDims, ParallelState
from relax_b200.rollout.weights import RolloutWeights, rollout_param_shapes
from relax_b200.weight_sync.plan import TrainerLayout, build_plan
from relax_b200.weight_sync.sync import apply_block


def _fake_ps(tp, rank):
    g1 = GroupInfo(None, (0,), 0)
    gt = GroupInfo(None, tuple(range(tp)), rank)
    return ParallelState(ParallelDims(tp=tp), rank, tuple(range(tp)), gt, g1, g1, g1, g1, g1, gt, gt)


def _hf_oracle(cfg, full):
    """Independent conversion of FULL Megatron-layout tensors to per-head q/k/v etc."""
    hd, ng = cfg.head_dim, cfg.num_query_groups
    qpg = cfg.num_attention_heads // ng
    out = {"embed": full["embedding.word_embeddings.weight"], "lm_head": full["output_layer.weight"],
           "final_norm": full["decoder.final_layernorm.weight"]}
    for i in range(cfg.num_layers):
        b = f"decoder.layers.{i}."
        qkv = full[b + "self_attention.linear_qkv.weight"].view(ng, qpg + 2, hd, cfg.hidden_size)
        out[f"{i}.q"] = qkv[:, :qpg].reshape(ng * qpg * hd, -1)
        out[f"{i}.k"] = qkv[:, qpg].reshape(ng * hd, -1)
        out[f"{i}.v"] = qkv[:, qpg + 1].reshape(ng * hd, -1)
        out[f"{i}.o"] = full[b + "self_attention.linear_proj.weight"]
        f1 = full[b + "mlp.linear_fc1.weight"]
        F = cfg.ffn_hidden_size
        out[f"{i}.gate"], out[f"{i}.up"] = f1[:F], f1[F:]
        out[f"{i}.down"] = full[b + "mlp.linear_fc2.weight"]
        out[f"{i}.in"] = full[b + "self_attention.linear_qkv.layer_norm_weight"]
        out[f"{i}.post"] = full[b + "mlp.linear_fc1.layer_norm_weight"]
        out[f"{i}.qn"] = full[b + "self_attention.q_layernorm.weight"]
        out[f"{i}.kn"] = full[b + "self_attention.k_layernorm.weight"]
    return out


def _expected_rollout_shard(cfg, hf, tp, r):
    sh = lambda t, dim: t.chunk(tp, dim)[r]
    exp = {"embed": sh(hf["embed"], 0), "lm_head": sh(hf["lm_head"], 0), "final_norm": hf["final_norm"]}
    for i in range(cfg.num_layers):
        p = f"layers.{i}."
        exp[p + "qkv"] = torch.cat([sh(hf[f"{i}.q"], 0), sh(hf[f"{i}.k"], 0), sh(hf[f"{i}.v"], 0)], 0)
        exp[p + "o"] = sh(hf[f"{i}.o"], 1)
        exp[p + "gate_up"] = torch.cat([sh(hf[f"{i}.gate"], 0), sh(hf[f"{i}.up"], 0)], 0)
        exp[p + "down"] = sh(hf[f"{i}.down"], 1)
        exp[p + "input_norm"], exp[p + "post_norm"] = hf[f"{i}.in"], hf[f"{i}.post"]
        exp[p + "q_norm"], exp[p + "k_norm"] = hf[f"{i}.qn"], hf[f"{i}.kn"]
    return exp


@pytest.mark.parametrize("src_tp,dst_tp", [(1, 1), (2, 2), (1, 2), (2, 1)])
def test_plan_matches_gather_convert_oracle(src_tp, dst_tp):
    cfg = get_config("tiny")
    # full model = TP1; shards = TP models of the same seed
    full = {k: v.detach() for k, v in GPTModel(cfg, _fake_ps(1, 0), seed=7).named_parameters()}
    shards = [{k: v.detach() for k, v in GPTModel(cfg, _fake_ps(src_tp, r), seed=7).named_parameters()}
              for r in range(src_tp)]
    # make norm weights non-trivial (they initialise to ones)
    torch.manual_seed(0)
    for k in full:
        if "norm" in k:
            nv = torch.randn_like(full[k])
            full[k].copy_(nv)
            for s in shards:
                s[k].copy_(nv)
    plan = build_plan(cfg, TrainerLayout(tp=src_tp), dst_tp)
    hf = _hf_oracle(cfg, full)
    shapes = rollout_param_shapes(cfg, dst_tp)
    covered = {r: {k: torch.zeros(s, dtype=torch.int32) for k, s in shapes.items()} for r in range(dst_tp)}
    for r in range(dst_tp):
        got = {k: torch.full(s, float("nan")) for k, s in shapes.items()}
        for b in plan:
            if b.dst_rank == r:
                apply_block(b, shards[b.src_rank][b.src_name], got[b.dst_name])
                ones = torch.ones(b.rows, b.cols, dtype=torch.int32)
                c = covered[r][b.dst_name]
                c = c.view(1, -1) if c.dim() == 1 else c
                c[b.dst_row:b.dst_row + b.rows, b.dst_col:b.dst_col + b.cols] += ones
        exp = _expected_rollout_shard(cfg, hf, dst_tp, r)
        for k in exp:
            assert torch.equal(got[k], exp[k]), k
        # every destination element written exactly once
        for k, c in covered[r].items():
            assert int(c.min()) == 1 and int(c.max()) == 1, k


def test_moe_plan_covers_experts():
    cfg = get_config("tiny-moe")
    plan = build_plan(cfg, TrainerLayout(tp=1, ep=2), 1, 2)
    names = {b.dst_name for b in plan}
    assert "layers.0.experts_gate_up" in names and "layers.1.router" in names
    per_dst = {}
    for b in plan:
        if b.dst_name == "layers.0.experts_gate_up":
            per_dst.setdefault(b.dst_rank, []).append((b.src_rank, b.src_batch, b.dst_batch))
    assert sorted(per_dst) == [0, 1] and all(len(v) == 4 for v in per_dst.values())
    assert per_dst[1][0] == (1, 0, 0)


def test_rollout_weights_roundtrip_through_sync_single_process():
    from relax_b200.weight_sync.sync import WeightSync

    cfg = get_config("tiny")
    model = GPTModel(cfg, seed=1)
    rw = RolloutWeights(cfg, 1, 0, "cpu", torch.float32)
    ws = WeightSync(cfg, TrainerLayout(), 1, [0], [0])
    ms = ws.update_weights(dict(model.named_parameters()), rw)
    assert ms >= 0
    hf = _hf_oracle(cfg, {k: v.detach() for k, v in model.named_parameters()})
    assert torch.equal(rw.p["layers.1.qkv"], torch.cat([hf["1.q"], hf["1.k"], hf["1.v"]], 0))
