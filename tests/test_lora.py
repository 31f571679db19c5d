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


def test_adapter_plan_reshards_factors_like_their_weights():
    """Adapter-mode sync: for trainer TP 2 -> rollout TP 1 and TP 2, base weight + scale * B A assembled from the
    synced factors on every rollout rank equals the rollout shard of the merged full weight (the oracle)."""
    from relax_b200.weight_sync.plan import TrainerLayout, build_adapter_plan, build_plan
    from relax_b200.weight_sync.sync import apply_block, oracle_rollout_state
    from relax_b200.rollout.weights import rollout_param_shapes

    cfg = get_config("tiny")
    r, scale = 4, 2.0
    g = torch.Generator().manual_seed(0)
    full = GPTModel(cfg, seed=3)
    LR.apply_lora(full, LR.LoRAConfig(rank=r, alpha=r * scale))
    for n, p in full.named_parameters():
        if "lora_" in n:
            p.data.copy_(torch.randn(p.shape, generator=g) * 0.1)
    merged_full = {n: p.detach() for n, p in LR.merged_named_params(full)}
    raw_full = {n: p.detach() for n, p in full.named_parameters()}
    for src_tp, dst_tp in ((1, 1), (2, 1), (2, 2), (1, 2)):
        # shard the raw trainer tensors (weights and factors) the way a TP-`src_tp` trainer holds them
        from relax_b200.parallel.state import GroupInfo, ParallelDims, ParallelState

        shards = []
        for tr in range(src_tp):
            one = GroupInfo(None, (0,), 0)
            ps = ParallelState(ParallelDims(tp=src_tp), tr, tuple(range(src_tp)), GroupInfo(None, tuple(range(src_tp)), tr),
                               one, one, one, one, one, one, one)
            m = GPTModel(cfg, ps, seed=3)
            LR.apply_lora(m, LR.LoRAConfig(rank=r, alpha=r * scale))
            from relax_b200.checkpoint.dist_ckpt import load_full_state

            load_full_state(cfg, ps, m, {k: v for k, v in raw_full.items() if "lora_" not in k}, strict=False)
            sh = {n: p.detach() for n, p in m.named_parameters()}
            # the factors in the layout train/lora.py gives them under TP: column-parallel linears (qkv, fc1) keep A
            # whole and B's rows of the rank's output features ([gate; up] halves for fc1); row-parallel ones (proj,
            # fc2) keep B whole and A's columns of the rank's input features
            for n in sh:
                if "lora_" not in n:
                    continue
                fullt = raw_full[n]
                col = ("linear_qkv" in n) or ("linear_fc1" in n)
                if n.endswith("lora_B") and col:
                    if "linear_fc1" in n:
                        F = fullt.shape[0] // 2
                        Fs = F // src_tp
                        sh[n] = torch.cat([fullt[tr * Fs:(tr + 1) * Fs], fullt[F + tr * Fs:F + (tr + 1) * Fs]])
                    else:
                        rows = fullt.shape[0] // src_tp
                        sh[n] = fullt[tr * rows:(tr + 1) * rows]
                elif n.endswith("lora_A") and not col:
                    cols = fullt.shape[1] // src_tp
                    sh[n] = fullt[:, tr * cols:(tr + 1) * cols]
                else:
                    sh[n] = fullt
                assert sh[n].shape == dict(m.named_parameters())[n].shape, n
            shards.append(sh)
        wplan = build_plan(cfg, TrainerLayout(tp=src_tp), dst_tp, 1)
        aplan = build_adapter_plan(cfg, TrainerLayout(tp=src_tp), dst_tp, r)
        for dr in range(dst_tp):
            shapes = rollout_param_shapes(cfg, dst_tp, 1)
            dst = {k: torch.zeros(s) for k, s in shapes.items()}
            for k, s in shapes.items():
                leaf = k.rsplit(".", 1)[-1]
                if k.startswith("layers.") and leaf in ("qkv", "o", "gate_up", "down"):
                    dst[k + ".lora_A"], dst[k + ".lora_B"] = torch.zeros(r, s[1]), torch.zeros(s[0], r)
            for b in wplan + aplan:
                if b.dst_rank == dr:
                    apply_block(b, shards[b.src_rank][b.src_name], dst[b.dst_name])
            want = oracle_rollout_state(cfg, merged_full, dst_tp, dr)
            for k in shapes:
                leaf = k.rsplit(".", 1)[-1]
                if k.startswith("layers.") and leaf in ("qkv", "o", "gate_up", "down"):
                    got = dst[k] + scale * dst[k + ".lora_B"] @ dst[k + ".lora_A"]
                    assert torch.allclose(got, want[k], atol=1e-5), (src_tp, dst_tp, dr, k)


def test_adapter_mode_sync_in_the_colocated_loop():
    """``--lora-adapter-mode``: after the first sync only the factors move, the engine adds them at run time and
    its log-probs keep matching the trainer's (adapted) forward."""
    from relax_b200.orchestration.colocate import ColocateConfig, ColocatedGRPO
    from relax_b200.weight_sync.plan import plan_bytes

    torch.manual_seed(0)
    cfg = ColocateConfig(
        model=get_config("tiny"),
        train=TrainConfig(n_samples_per_prompt=2, global_batch_size=8, max_tokens_per_gpu=1024, lora=LR.LoRAConfig(rank=4, alpha=8),
                          loss=LossConfig(), optim=OptimizerConfig(lr=5e-3, weight_decay=0.0)),
        rollout_batch_size=4, prompt_len=8, max_response_len=12, rm_type="parity", lora_adapter_mode=True, seed=0, rollout_seed=1,
        stop_token_ids=list(range(0, 1024, 6)))        # responses of different lengths: the parity reward varies inside groups
    run = ColocatedGRPO(cfg)
    assert run.engine.weights.lora and run._base_synced is False or run._base_synced is True
    for _ in range(3):
        m = run.step()
        assert m["train_rollout_logprob_abs_diff"] < 1e-4
    assert run._base_synced
    b_name = next(k for k in run.engine.weights.lora if k.endswith("qkv.lora_B"))
    assert run.engine.weights.lora[b_name].abs().sum() > 0, "the factors reached the engine"
    small = plan_bytes(run.adapter_syncs[0][0].plan)
    assert small * 10 < plan_bytes(run.syncs[0][0].plan), "an adapter sync moves a fraction of a full sync"
    run.close()
