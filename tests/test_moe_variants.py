"""DeepSeek-V3 / GLM4-MoE / Qwen2-MoE style MoE pieces: sigmoid routing with a selection bias, shared expert (optionally
gated), leading dense layers; trainer <-> rollout weight plan and HF names (CPU)."""
import torch

from relax_b200.checkpoint import hf as H
from relax_b200.models.config import get_config
from relax_b200.models.moe import MoEMLP, route_tokens
from relax_b200.models.transformer import GPTModel
from relax_b200.rollout.weights import RolloutWeights
from relax_b200.weight_sync.plan import TrainerLayout
from relax_b200.weight_sync.sync import WeightSync


def test_sigmoid_routing_selects_on_biased_scores_but_weights_plain_ones():
    cfg = get_config("tiny-dsv3")
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, -2.0, -3.0, -4.0, -5.0]])
    w, idx, sc = route_tokens(logits, cfg, None)
    assert sorted(idx[0].tolist()) == [0, 1]
    s = torch.sigmoid(logits[0, :2])
    assert torch.allclose(w[0].sort().values, (s / s.sum() * 2.5).sort().values, atol=1e-6)
    bias = torch.zeros(8)
    bias[7] = 5.0
    w2, idx2, _ = route_tokens(logits, cfg, bias)
    assert 7 in idx2[0].tolist() and 0 in idx2[0].tolist()
    j = idx2[0].tolist().index(7)
    s7, s0 = torch.sigmoid(logits[0, 7]), torch.sigmoid(logits[0, 0])
    assert torch.allclose(w2[0, j], s7 / (s7 + s0) * 2.5, atol=1e-6)     # the bias never enters the weight


def test_bias_update_moves_towards_even_load():
    cfg = get_config("tiny-dsv3")
    m = GPTModel(cfg, seed=0)
    moe = m.decoder.layers[1].mlp
    assert isinstance(moe, MoEMLP) and not moe.router.expert_bias.requires_grad
    m.train()
    toks = torch.randint(3, 1000, (64,), generator=torch.Generator().manual_seed(0))
    m(toks, torch.arange(64), torch.tensor([0, 64], dtype=torch.int32))
    c = moe.last_counts.clone().float()
    moe.update_router_bias(0.01)
    b = moe.router.expert_bias
    assert (b[c < c.mean()] > 0).all() and (b[c > c.mean()] < 0).all() and moe.last_counts is None


def test_dense_first_layer_shared_expert_and_grads():
    cfg = get_config("tiny-dsv3", moe_shared_expert_gate=True)
    m = GPTModel(cfg, seed=1)
    assert not m.decoder.layers[0].is_moe_layer and m.decoder.layers[1].is_moe_layer
    toks = torch.arange(10) + 5
    h = m(toks, torch.arange(10), torch.tensor([0, 10], dtype=torch.int32))
    lp, _ = m.log_probs(h[:-1], toks[1:], with_entropy=False)
    lp.sum().backward()
    se = m.decoder.layers[1].mlp.shared_experts
    assert se.linear_fc1.weight.grad.abs().sum() > 0 and se.gate_weight.grad.abs().sum() > 0
    assert m.decoder.layers[1].mlp.router.expert_bias.grad is None


def test_rollout_weights_match_trainer_forward_after_sync():
    cfg = get_config("tiny-dsv3", moe_shared_expert_gate=True)
    m = GPTModel(cfg, seed=2)
    with torch.no_grad():
        for l in m.decoder.layers[1:]:
            l.mlp.router.expert_bias.copy_(torch.linspace(-0.3, 0.3, cfg.num_experts))
    rw = RolloutWeights(cfg, 1, 0, "cpu", torch.float32)
    ws = WeightSync(cfg, TrainerLayout(), 1, [0], [0])
    ws.update_weights(dict(m.named_parameters()), rw)
    toks = torch.arange(12) + 7
    pos = torch.arange(12)
    cu = torch.tensor([0, 12], dtype=torch.int32)
    with torch.no_grad():
        ref = m.logits(m(toks, pos, cu))

        def attn(i, q, k, v):
            from relax_b200 import ops
            return ops.attention_varlen(q, k, v, cu, causal=True)

        nl = cfg.num_layers
        kv = torch.zeros(nl, 2, 4, 16, cfg.num_query_groups, cfg.head_dim)
        from relax_b200.parallel.state import single_process_state
        out = rw.forward_prefill(toks, pos, cu, torch.arange(12), kv, torch.arange(12), single_process_state().tp)
    assert torch.allclose(out, ref.float(), atol=2e-3), (out - ref).abs().max()


def test_hf_names_roundtrip():
    for gate in (False, True):
        cfg = get_config("tiny-dsv3", moe_shared_expert_gate=gate)
        m = GPTModel(cfg, seed=3)
        state = {k: v.detach() for k, v in m.named_parameters()}
        hf = H.convert_state_to_hf(cfg, state)
        sh = "shared_expert" if gate else "shared_experts"
        assert f"model.layers.1.mlp.{sh}.gate_proj.weight" in hf and "model.layers.1.mlp.gate.e_score_correction_bias" in hf
        assert ("model.layers.1.mlp.shared_expert_gate.weight" in hf) == gate
        assert "model.layers.0.mlp.gate_proj.weight" in hf and "model.layers.0.mlp.gate.weight" not in hf
        back = H.hf_to_megatron_state(cfg, hf)
        assert set(back) == set(state) and all(torch.equal(back[k], state[k]) for k in state)
        d = H.hf_config_dict(cfg)
        assert d["first_k_dense_replace"] == 1 and d["scoring_func"] == "sigmoid" and d["n_shared_experts"] == 1


def test_trainer_updates_router_bias_each_step():
    from relax_b200.algo.loss import LossConfig
    from relax_b200.train.actor import TrainActor, TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    torch.manual_seed(0)
    actor = TrainActor(get_config("tiny-dsv3"), TrainConfig(global_batch_size=2, max_tokens_per_gpu=64, pad_multiple=1,
                       loss=LossConfig(), optim=OptimizerConfig(lr=1e-3, weight_decay=0.0)), role="sft")
    actor.model.train()
    b = {"tokens": [[5, 6, 7, 8, 9, 10, 11, 12], [11, 12, 13, 14, 15, 16]], "response_lengths": [4, 3],
         "loss_masks": [[1.0] * 4, [1.0] * 3]}
    actor.train_sft(b)
    bias = actor.model.decoder.layers[1].mlp.router.expert_bias
    assert float(bias.abs().max()) > 0 and abs(float(bias.abs().max()) - 1e-3) < 1e-6
