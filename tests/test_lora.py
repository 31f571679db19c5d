"""LoRA: adapters only are trained, merged weights reproduce the adapted forward, TP layout agrees with TP1."""
import torch

from relax_b200.algo.loss import LossConfig
from relax_b200.models.config import get_config
from relax_b200.models.transformer import GPTModel
from relax_b200.train import lora as LR
from relax_b200.train.actor import TrainActor, TrainConfig
from relax_b200.train.optimizer import OptimizerConfig
from tests._mp import run_distributed


def _batch():
    toks = [[5, 6, 7, 8, 9, 10, 11, 12], [11, 12, 13, 14, 15, 16]]
    rl = [4, 3]
    return {"tokens": toks, "response_lengths": rl, "loss_masks": [[1.0] * r for r in rl]}


def test_lora_trains_adapters_only_and_merges():
    torch.manual_seed(0)
    cfg = TrainConfig(global_batch_size=2, max_tokens_per_gpu=64, pad_multiple=1, lora=LR.LoRAConfig(rank=4, alpha=8),
                      loss=LossConfig(), optim=OptimizerConfig(lr=5e-3, weight_decay=0.0))
    actor = TrainActor(get_config("tiny"), cfg, role="sft", with_reference=True)
    base = {n: p.detach().clone() for n, p in actor.model.named_parameters() if "lora" not in n}
    trainable = [n for n, p in actor.model.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable)
    b = _batch()
    nll0 = actor.evaluate_ppl(b)["eval/nll"]
    for _ in range(6):
        actor.train_sft(b)
    assert actor.evaluate_ppl(b)["eval/nll"] < nll0 - 0.2
    for n, p in actor.model.named_parameters():
        if "lora" not in n:
            assert torch.equal(p, base[n]), n      # frozen
    # reference snapshot = adapters at their initial value (B = 0) = the base model
    ref_lp = actor.compute_log_prob(b, "ref")["log_probs"]
    plain = TrainActor(get_config("tiny"), TrainConfig(pad_multiple=1), with_optimizer=False)
    for x, y in zip(plain.compute_log_prob(b)["log_probs"], ref_lp):
        assert torch.allclose(x, y, atol=1e-5)
    # merged weights in a plain model reproduce the adapted model
    lp_adapted = actor.compute_log_prob(b)["log_probs"]
    merged = dict(actor.named_local_params())
    with torch.no_grad():
        for n, p in plain.model.named_parameters():
            p.copy_(merged[n])
    for x, y in zip(lp_adapted, plain.compute_log_prob(b)["log_probs"]):
        assert torch.allclose(x, y, atol=2e-4)
    sd = LR.adapter_state_dict(actor.model)
    fp = LR.adapter_fingerprint(actor.model)
    assert fp > 0 and len(sd) == 2 * 4 * get_config("tiny").num_layers
    LR.merge_and_unload(actor.model)
    assert not any("lora" in n for n, _ in actor.model.named_parameters())


def _tp_worker(rank, world):
    from relax_b200.parallel.state import ParallelDims, init_parallel_state

    ps = init_parallel_state(ParallelDims(tp=2))
    cfg = get_config("tiny")
    m = GPTModel(cfg, ps, seed=3)
    LR.apply_lora(m, LR.LoRAConfig(rank=4, alpha=8, seed=5))
    g = torch.Generator().manual_seed(9)
    with torch.no_grad():
        for n, mod in m.named_modules():
            if hasattr(mod, "lora_B"):
                full_out = mod.lora_B.shape[0] * (2 if n.rsplit(".", 1)[-1] in ("linear_qkv", "linear_fc1") else 1)
                fb = torch.randn(full_out, 4, generator=g) * 0.1
                if mod.lora_B.shape[0] != full_out:
                    rows = mod.lora_B.shape[0]
                    if n.endswith("linear_fc1"):   # [gate; up] halves are sharded separately
                        h = full_out // 2
                        fb = torch.cat([fb[rank * rows // 2:(rank + 1) * rows // 2], fb[h + rank * rows // 2: h + (rank + 1) * rows // 2]])
                    else:
                        fb = fb[rank * rows:(rank + 1) * rows]
                mod.lora_B.copy_(fb)
    toks = torch.arange(8) + 3
    pos = torch.arange(8)
    cu = torch.tensor([0, 8], dtype=torch.int32)
    h = m(toks, pos, cu)
    lp, _ = m.log_probs(h[:-1], toks[1:], with_entropy=False)
    lp.sum().backward()
    ga = m.decoder.layers[0].self_attention.linear_qkv.lora_A.grad
    return lp.detach(), ga.detach()


def test_lora_forward_runs_under_tp2_and_is_rank_consistent():
    out = run_distributed(_tp_worker, 2)
    assert torch.allclose(out[0][0], out[1][0], atol=1e-5)   # both ranks compute the same log-probs
    assert out[0][1].abs().sum() > 0
