"""Multi-token-prediction blocks and the sequence-classification head (CPU, tiny model)."""
import math

import torch

from relax_b200.algo.loss import LossConfig
from relax_b200.models.config import get_config
from relax_b200.models.mtp import mtp_forward, shift_in_sequence
from relax_b200.models.transformer import GPTModel
from relax_b200.train.actor import TrainActor, TrainConfig, _shift_mask
from relax_b200.train.optimizer import OptimizerConfig
from tests._mp import run_distributed


def test_shift_stays_inside_sequences():
    toks = torch.tensor([1, 2, 3, 4, 5, 6, 7, 0, 0])
    cu = torch.tensor([0, 3, 7, 9], dtype=torch.int32)
    s1, ok1 = shift_in_sequence(toks, cu, 1)
    assert s1.tolist() == [2, 3, 0, 5, 6, 7, 0, 0, 0]
    assert ok1.tolist() == [True, True, False, True, True, True, False, True, False]
    s2, ok2 = shift_in_sequence(toks, cu, 2)
    assert s2.tolist() == [3, 0, 0, 6, 7, 0, 0, 0, 0] and ok2.tolist()[:7] == [True, False, False, True, True, False, False]
    m = torch.tensor([1., 1., 0., 1., 1.])
    assert _shift_mask(m, [3, 2], 1).tolist() == [1., 0., 0., 1., 0.]


def _batch():
    toks = [[5, 6, 7, 8, 9, 10, 11, 12], [11, 12, 13, 14, 15, 16]]
    rl = [5, 4]
    return {"tokens": toks, "response_lengths": rl, "loss_masks": [[1.0] * r for r in rl]}


def _cfg(**kw):
    return TrainConfig(global_batch_size=2, max_tokens_per_gpu=64, pad_multiple=1, loss=LossConfig(),
                       optim=OptimizerConfig(lr=3e-3, weight_decay=0.0), **kw)


def test_mtp_loss_matches_manual_cross_entropy():
    cfg = get_config("tiny", mtp_num_layers=2)
    m = GPTModel(cfg, seed=1)
    toks = torch.tensor([5, 6, 7, 8, 9, 10, 3, 4, 5, 6])
    pos = torch.cat([torch.arange(6), torch.arange(4)])
    cu = torch.tensor([0, 6, 10], dtype=torch.int32)
    h, pre = m(toks, pos, cu, return_prenorm=True)
    rows = torch.arange(10)
    out = mtp_forward(m, pre, toks, pos, cu, rows)
    assert len(out) == 2
    (lp1, ok1), (lp2, ok2) = out
    assert ok1.tolist() == [True] * 4 + [False] * 2 + [True] * 2 + [False] * 2
    assert ok2.tolist() == [True] * 3 + [False] * 3 + [True] * 1 + [False] * 3
    # depth 1 by hand: block(prenorm, emb(t+1)) -> shared head -> log p(t+2)
    blk = m.mtp.layers[0]
    t1, _ = shift_in_sequence(toks, cu, 1)
    t2, _ = shift_in_sequence(toks, cu, 2)
    cos, sin = m.rope_tables(pos)
    _, hn = blk(pre, m.embedding.word_embeddings(t1, False), cos, sin, cu)
    ref = torch.log_softmax(hn.float() @ m.lm_head_weight().float().t(), -1).gather(1, t2[:, None])[:, 0]
    assert torch.allclose(lp1[ok1], ref[ok1], atol=1e-4)
    assert torch.isfinite(lp2).all()


def test_mtp_training_adds_loss_and_learns():
    torch.manual_seed(0)
    actor = TrainActor(get_config("tiny", mtp_num_layers=1), _cfg(enable_mtp_training=True, mtp_loss_scaling_factor=0.3), role="sft")
    b = _batch()
    first = actor.train_sft(b)
    for _ in range(10):
        last = actor.train_sft(b)
    assert "mtp_loss" in first and last["mtp_loss"] < first["mtp_loss"] * 0.7 and last["loss"] < first["loss"]
    assert math.isfinite(last["grad_norm"])
    # the policy-gradient role takes the same extra term
    pol = TrainActor(get_config("tiny", mtp_num_layers=1), _cfg(enable_mtp_training=True), role="actor")
    pb = dict(b, advantages=[[0.5] * r for r in b["response_lengths"]],
              log_probs=[[-1.0] * r for r in b["response_lengths"]])
    out, _ = pol._train_step(pb, [0, 1])
    assert "mtp_loss" in out and "pg_loss" in out


def test_mtp_only_training_freezes_trunk():
    torch.manual_seed(0)
    actor = TrainActor(get_config("tiny", mtp_num_layers=1), _cfg(mtp_only_training=True), role="sft")
    before = {n: p.detach().clone() for n, p in actor.model.named_parameters()}
    m0 = actor.train_sft(_batch())
    for _ in range(5):
        m1 = actor.train_sft(_batch())
    changed = {n for n, p in actor.model.named_parameters() if not torch.equal(p, before[n])}
    assert changed and all(n.startswith("mtp.") for n in changed)
    assert m1["mtp_loss"] < m0["mtp_loss"]


def _tp_worker(rank, world):
    from relax_b200.parallel.state import ParallelDims, init_parallel_state

    ps = init_parallel_state(ParallelDims(tp=2))
    m = GPTModel(get_config("tiny", mtp_num_layers=1), ps, seed=4)
    toks = torch.arange(8) + 3
    pos = torch.arange(8)
    cu = torch.tensor([0, 8], dtype=torch.int32)
    h, pre = m(toks, pos, cu, return_prenorm=True)
    (lp, ok), = mtp_forward(m, pre, toks, pos, cu, torch.arange(8))
    (lp * ok).sum().backward()
    return lp.detach(), ok, m.mtp.layers[0].eh_proj.weight.grad.detach()


def test_mtp_under_tp2_matches_single_rank():
    out = run_distributed(_tp_worker, 2)
    m = GPTModel(get_config("tiny", mtp_num_layers=1), seed=4)
    toks = torch.arange(8) + 3
    pos = torch.arange(8)
    cu = torch.tensor([0, 8], dtype=torch.int32)
    h, pre = m(toks, pos, cu, return_prenorm=True)
    (lp, ok), = mtp_forward(m, pre, toks, pos, cu, torch.arange(8))
    (lp * ok).sum().backward()
    assert torch.allclose(out[0][0][ok], lp.detach()[ok], atol=1e-4) and torch.allclose(out[1][0][ok], lp.detach()[ok], atol=1e-4)
    # replicated projection: the two sequence-parallel partial gradients add up to the full one
    assert torch.allclose(out[0][2] + out[1][2], m.mtp.layers[0].eh_proj.weight.grad, atol=1e-4)


def test_sequence_classification_head_learns():
    torch.manual_seed(0)
    actor = TrainActor(get_config("tiny", num_classes=3), _cfg(), role="seq_cls")
    toks = [[5, 6, 7, 8], [9, 10, 11, 12, 13], [20, 21, 22], [30, 31, 32, 33, 34, 35]]
    batch = {"tokens": toks, "response_lengths": [1] * 4, "labels": [0, 1, 2, 1]}
    first = actor.train_seq_cls(batch)
    for _ in range(15):
        last = actor.train_seq_cls(batch)
    assert last["loss"] < first["loss"] * 0.5 and last["accuracy"] == 1.0
    pred = [int(r.argmax()) for r in actor.predict_classes(batch)]
    assert pred == batch["labels"]


def test_mtp_parameters_round_trip_through_hf_names():
    from relax_b200.checkpoint import hf as H

    cfg = get_config("tiny", mtp_num_layers=2)
    m = GPTModel(cfg, seed=6)
    state = {k: v.detach() for k, v in m.named_parameters()}
    hf = H.convert_state_to_hf(cfg, state)
    L = cfg.num_layers
    assert f"model.layers.{L}.eh_proj.weight" in hf and f"model.layers.{L + 1}.shared_head.norm.weight" in hf
    assert f"model.layers.{L}.self_attn.q_proj.weight" in hf and f"model.layers.{L}.mlp.down_proj.weight" in hf
    back = H.hf_to_megatron_state(cfg, hf)
    assert set(back) == set(state) and all(torch.equal(back[k], state[k]) for k in state)
