"""Trainer and rollout pools in different processes (gloo, CPU): role placement from ``--resource``, batches through
the queue service, bounded staleness, and weights written by the trainer process straight into the rollout
processes' parameter buffers (shared memory standing in for NVLink peer mappings) - against the broadcast arm and
a gather-then-convert oracle."""
import os

import pytest
import torch

from tests._mp import run_distributed


def _worker(rank, world, push, trainer_tp, rollout_tp, n_train, port_tag, num_iters=1, speculative=False, model="tiny"):
    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.orchestration.disagg import DisaggConfig, DisaggregatedRL
    from relax_b200.orchestration.registry import assign_ranks
    from relax_b200.train.actor import TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig
    from relax_b200.weight_sync.sync import oracle_rollout_state

    ranks = assign_ranks({"actor": (1, n_train), "rollout": (1, world - n_train)}, world, colocate=False)
    assert ranks["actor"] == tuple(range(n_train)) and ranks["rollout"] == tuple(range(n_train, world))
    mcfg = get_config(model, mtp_num_layers=1) if speculative else get_config(model)
    cfg = DisaggConfig(
        model=mcfg, train=TrainConfig(n_samples_per_prompt=2, global_batch_size=8, pad_multiple=1, max_tokens_per_gpu=512,
                                      loss=LossConfig(use_kl_loss=True, kl_loss_coef=0.001), optim=OptimizerConfig(lr=1e-2)),
        trainer_ranks=ranks["actor"], rollout_ranks=ranks["rollout"], trainer_tp=trainer_tp, rollout_tp=rollout_tp,
        rollout_batch_size=4, prompt_len=8, max_response_len=6, kv_blocks=64, kv_block_size=4, num_rollout=3, max_staleness=1,
        weight_push=push, tag=f"t{port_tag}", handshake_timeout_s=120.0, num_iters_per_train_update=num_iters,
        speculative=speculative, speculative_steps=2)
    run = DisaggregatedRL(cfg, device="cpu")
    out = run.run()
    res = {"role": "actor" if run.is_trainer else "rollout"}
    import torch.distributed as dist

    if run.is_trainer:
        res["metrics"] = [(rid, {k: float(v) for k, v in m.items()}) for rid, m in out]
        res["stats"] = {k: v for k, v in run.stats.items() if isinstance(v, (int, float))}
        res["mtp"] = {k: v.detach().numpy().copy() for k, v in run.actor.named_local_params() if k.startswith("mtp.layers.0.eh_proj")}
        res["version"] = run.actor.weight_version
        res["params"] = {k: v.detach().numpy().copy() for k, v in run.actor.named_local_params()} if trainer_tp == 1 else None
    else:
        res["started"] = run.stats["rollout_started"]
        res["version"] = run.engine.weight_version
        res["weights"] = {k: v.numpy().copy() for k, v in run.engine.weights.p.items()}
        res["tp_rank"] = run.engine.tp.rank
        res["spec"] = {k: run.engine.stats.get(k, 0) for k in ("spec_draft_tokens", "spec_verify_steps")}
    dist.barrier()
    run.close()
    return res


@pytest.mark.parametrize("push", ["peer", "broadcast"])
def test_disjoint_pools_run_and_engines_end_with_the_trainers_weights(push):
    from relax_b200.models.config import get_config
    from relax_b200.weight_sync.sync import oracle_rollout_state

    out = run_distributed(_worker, 3, push, 1, 1, 1, os.getpid() % 10000 + (1 if push == "peer" else 2), timeout=600)
    tr = [o for o in out if o["role"] == "actor"][0]
    ro = [o for o in out if o["role"] == "rollout"]
    assert len(tr["metrics"]) == 3 and tr["version"] == 3
    assert all("loss" in m and m["response_tokens"] > 0 for _, m in tr["metrics"])
    assert 0.0 <= tr["stats"]["trainer_idle_fraction"] <= 1.0 and tr["stats"]["tokens_per_s"] > 0
    cfg = get_config("tiny")
    for o in ro:
        assert o["version"] == 3
        # generation never ran more than max_staleness + 1 rollouts ahead of the weights it had
        for rid, v in o["started"]:
            assert rid - v <= 2, o["started"]
        want = oracle_rollout_state(cfg, {k: torch.from_numpy(v) for k, v in tr["params"].items()}, 1, 0)
        for k, w in want.items():
            assert torch.equal(torch.from_numpy(o["weights"][k]), w), k


def test_disjoint_pools_trainer_tp2_to_rollout_tp2_by_peer_stores():
    """Four processes: trainer TP2 on ranks 0-1, one TP2 engine on ranks 2-3; every trainer rank writes its shard's
    blocks into both engine ranks' buffers."""
    out = run_distributed(_worker, 4, "peer", 2, 2, 2, os.getpid() % 10000 + 3, timeout=600)
    tr = [o for o in out if o["role"] == "actor"]
    ro = [o for o in out if o["role"] == "rollout"]
    assert len(tr) == 2 and len(ro) == 2 and all(o["version"] == 3 for o in ro)
    assert sorted(o["tp_rank"] for o in ro) == [0, 1]
    # both engine ranks received finite, non-trivial weights and differ where the shards differ
    a, b = ({k: torch.from_numpy(v) for k, v in o["weights"].items()} for o in ro)
    assert all(torch.isfinite(v).all() for v in a.values())
    assert not torch.equal(a["layers.0.qkv"], b["layers.0.qkv"]) and torch.equal(a["final_norm"], b["final_norm"])


def test_disjoint_pools_trainer_tp2_broadcast_arm():
    out = run_distributed(_worker, 4, "broadcast", 2, 2, 2, os.getpid() % 10000 + 4, timeout=600)
    ro = [o for o in out if o["role"] == "rollout"]
    assert len(ro) == 2 and all(o["version"] == 3 for o in ro)


def _vl_worker(rank, world, port_tag):
    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.orchestration.disagg import DisaggConfig, DisaggregatedRL
    from relax_b200.train.actor import TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    cfg = DisaggConfig(
        model=get_config("tiny-vl"),
        train=TrainConfig(n_samples_per_prompt=2, global_batch_size=8, pad_multiple=1, max_tokens_per_gpu=1024,
                          freeze_params_name_list=[r"^vision\."], loss=LossConfig(use_kl_loss=True, kl_loss_coef=0.001),
                          optim=OptimizerConfig(lr=1e-2)),
        trainer_ranks=(0,), rollout_ranks=(1,), trainer_tp=1, rollout_tp=1, rollout_batch_size=4, prompt_len=24, max_response_len=6,
        kv_blocks=128, kv_block_size=4, num_rollout=2, max_staleness=1, weight_push="peer", tag=f"v{port_tag}", handshake_timeout_s=120.0)
    run = DisaggregatedRL(cfg, device="cpu")
    out = run.run()
    import torch.distributed as dist

    res = {"role": "actor" if run.is_trainer else "rollout"}
    if run.is_trainer:
        res["metrics"] = [(rid, {k: float(v) for k, v in m.items()}) for rid, m in out]
    dist.barrier()
    run.close()
    return res


def test_vision_language_on_disjoint_pools():
    """Config-3 shape on the CPU: image prompts generated by an engine process with its own (frozen) tower, batches with
    the patches through the queue service, trained by another process; log-probs of the two sides agree."""
    out = run_distributed(_vl_worker, 2, os.getpid() % 10000 + 7, timeout=600)
    tr = [o for o in out if o["role"] == "actor"][0]
    assert len(tr["metrics"]) == 2
    assert all(m["response_tokens"] > 0 for _, m in tr["metrics"])
    # the first rollout was generated with the weights the trainer still holds (later ones may be one version behind)
    assert tr["metrics"][0][1]["train_rollout_logprob_abs_diff"] < 1e-3


def test_streamed_parts_forward_early_and_train_like_the_whole_batch():
    """``num_iters_per_train_update`` = 2: the engine publishes finished prompt groups early, the trainer runs its
    forward-only passes per part, and the optimizer steps see the same rows as in the unsplit run (one engine, so
    both runs generate the same samples): losses agree, engines end with the trainer's weights."""
    whole = run_distributed(_worker, 2, "peer", 1, 1, 1, os.getpid() % 10000 + 7, timeout=600)
    parts = run_distributed(_worker, 2, "peer", 1, 1, 1, os.getpid() % 10000 + 8, 2, timeout=600)
    a = [o for o in whole if o["role"] == "actor"][0]
    b = [o for o in parts if o["role"] == "actor"][0]
    assert b["stats"]["parts_forwarded"] >= 2 * 3 and "parts_forwarded" not in a["stats"]
    assert b["version"] == 3 and [o for o in parts if o["role"] == "rollout"][0]["version"] == 3
    for (_, ma), (_, mb) in zip(a["metrics"][:1], b["metrics"][:1]):          # later rollouts depend on the overlap timing
        assert ma["response_tokens"] == mb["response_tokens"]
        assert abs(ma["loss"] - mb["loss"]) < 1e-4 and abs(ma["grad_norm"] - mb["grad_norm"]) < 1e-3 * max(1.0, ma["grad_norm"])


@pytest.mark.parametrize("push", ["peer", "broadcast"])
def test_speculating_engines_on_disjoint_pools(push):
    """Fully-async with engines that draft with the MTP block: the block's weights are pushed with the policy's (peer
    stores and the broadcast arm) and the engines speculate with them."""
    out = run_distributed(_worker, 2, push, 1, 1, 1, os.getpid() % 10000 + (11 if push == "peer" else 12), 1, True, timeout=600)
    tr = [o for o in out if o["role"] == "actor"][0]
    ro = [o for o in out if o["role"] == "rollout"][0]
    assert tr["version"] == 3 and ro["version"] == 3 and ro["spec"]["spec_draft_tokens"] > 0 and ro["spec"]["spec_verify_steps"] > 0
    assert torch.equal(torch.from_numpy(ro["weights"]["mtp.eh_proj"]), torch.from_numpy(tr["mtp"]["mtp.layers.0.eh_proj.weight"]))


@pytest.mark.parametrize("model", ["tiny-qwen35", "tiny-dsa"])
def test_hybrid_and_latent_families_on_disjoint_pools(model):
    """Fully-async with a Gated-DeltaNet hybrid and with sparse latent attention: the engines serve the family and end
    with the trainer's weights (the extra tensors travel through the same peer stores)."""
    from relax_b200.models.config import get_config
    from relax_b200.weight_sync.sync import oracle_rollout_state

    out = run_distributed(_worker, 2, "peer", 1, 1, 1, os.getpid() % 10000 + (21 if model == "tiny-dsa" else 22), 1, False, model, timeout=600)
    tr = [o for o in out if o["role"] == "actor"][0]
    ro = [o for o in out if o["role"] == "rollout"][0]
    assert tr["version"] == 3 and ro["version"] == 3 and all("loss" in m for _, m in tr["metrics"])
    want = oracle_rollout_state(get_config(model), {k: torch.from_numpy(v) for k, v in tr["params"].items()}, 1, 0)
    assert set(want) == set(ro["weights"])
    for k, w in want.items():
        assert torch.equal(torch.from_numpy(ro["weights"][k]), w), k
