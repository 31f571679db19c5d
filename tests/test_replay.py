"""Trajectory replay: capture the loss / advantage stages, replay them, detect a changed implementation."""
import torch

from relax_b200.algo import loss as L
from relax_b200.algo.ppo_utils import Segments
from relax_b200.utils.replay import ReplayRecorder, default_stage_functions, replay_bundle


def _loss_inputs():
    torch.manual_seed(0)
    seg = Segments.from_lengths([3, 2])
    lp = torch.randn(5) * 0.1 - 1.0
    b = L.LossBatch(seg=seg, loss_mask=torch.ones(5), advantages=torch.randn(5), old_log_probs=lp + 0.05 * torch.randn(5),
                    ref_log_probs=lp.clone(), rollout_log_probs=None, returns=None, values=None, sample_denoms=None)
    return dict(log_probs=lp, entropy=torch.rand(5), batch=b, cfg=L.LossConfig(eps_clip=0.2, use_kl_loss=True, kl_loss_coef=0.01))


def test_capture_and_replay_roundtrip(tmp_path):
    rec = ReplayRecorder(str(tmp_path))
    fns = default_stage_functions()
    run_loss = rec.wrap("loss", fns["loss"], lambda: 3)
    out = run_loss(**_loss_inputs())
    adv_in = dict(estimator="grpo", rewards=torch.tensor([1.0, 0.0]), seg=Segments.from_lengths([3, 2]), loss_mask=torch.ones(5))
    rec.wrap("advantages", fns["advantages"], lambda: 3)(**adv_in)
    assert len(rec.records) == 2 and rec.records[0]["rollout_id"] == 3
    reports = replay_bundle(str(tmp_path))
    assert [r["ok"] for r in reports] == [True, True]
    # a changed implementation is flagged with the path of the first difference
    bad = dict(fns)
    bad["loss"] = lambda **kw: {"loss": fns["loss"](**kw)["loss"] * 1.01, "metrics": fns["loss"](**kw)["metrics"]}
    rep = {r["stage"]: r for r in replay_bundle(str(tmp_path), bad)}       # reports come in run order: advantages, then loss
    assert rep["loss"]["ok"] is False and rep["loss"]["diffs"][0][0] == "out.loss" and rep["advantages"]["ok"]
    assert torch.is_tensor(out["loss"])


def test_disabled_recorder_is_free(tmp_path):
    rec = ReplayRecorder(None)
    assert rec.capture("loss", 0, {}, {}) is None and not rec.enabled
    small = ReplayRecorder(str(tmp_path), stages=("loss",), max_records=1)
    assert small.capture("advantages", 0, {}, {}) is None
    assert small.capture("loss", 0, {"x": torch.ones(1)}, {"y": 1.0}) is not None
    assert small.capture("loss", 1, {"x": torch.ones(1)}, {"y": 1.0}) is None


def test_routing_replay_in_the_trainer_survives_different_microbatching():
    """The old-policy forward packs all samples in one micro-batch, the training steps pack them two at a time: the
    per-sample store re-assembles the recorded expert choices, and the first training forward reproduces the
    old-policy log-probs exactly (ratio 1) even though a perturbed router would choose differently."""
    import torch
    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.models.moe import RoutingReplay
    from relax_b200.train.actor import TrainActor, TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    torch.manual_seed(0)
    cfg = TrainConfig(advantage_estimator="grpo", global_batch_size=2, n_samples_per_prompt=2, max_tokens_per_gpu=1024, pad_multiple=1,
                      use_routing_replay=True, loss=LossConfig(), optim=OptimizerConfig(lr=0.0))
    actor = TrainActor(get_config("tiny-moe"), cfg, role="actor")
    g = torch.Generator().manual_seed(1)
    toks = [torch.randint(3, 1000, (n,), generator=g).tolist() for n in (12, 9, 14, 10)]
    rl = [5, 4, 6, 3]
    batch = {"tokens": toks, "response_lengths": rl, "loss_masks": [[1.0] * r for r in rl], "rewards": [1.0, 0.0, 0.0, 1.0]}
    seen = []
    orig = RoutingReplay.route.__func__

    def spy(cls, layer, idx):
        out = orig(cls, layer, idx)
        seen.append((cls.mode, layer, idx.shape[0], bool((out != idx).any()) if out.shape == idx.shape else None))
        return out

    RoutingReplay.route = classmethod(spy)
    try:
        m = actor.train(0, batch)
    finally:
        RoutingReplay.route = classmethod(orig)
    modes = [s[0] for s in seen]
    assert "record" in modes and "replay" in modes and RoutingReplay.mode is None
    rec_rows = {s[2] for s in seen if s[0] == "record"}
    rep_rows = {s[2] for s in seen if s[0] == "replay"}
    assert rec_rows == {45} and rep_rows == {21, 24}            # one micro-batch of 4 samples vs two steps of 2
    assert abs(m["ppo_kl"]) < 1e-6 and m["pg_clipfrac"] == 0.0


def test_rollout_routing_replay_r3_engine_choices_drive_the_trainer():
    """R3: the engine returns, per fed position, the experts every MoE layer chose; with ``use_rollout_routing_replay``
    the trainer's old-policy and training forwards replay exactly those choices (a spy on the router sees the recorded
    ids come back), both through the host-driven and the windowed decode loop."""
    import torch
    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.models.moe import RoutingReplay
    from relax_b200.rollout.engine import RolloutEngine, SamplingParams
    from relax_b200.train.actor import TrainActor, TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig
    from relax_b200.weight_sync.plan import TrainerLayout
    from relax_b200.weight_sync.sync import WeightSync

    mcfg = get_config("tiny-moe")
    cfg = TrainConfig(advantage_estimator="grpo", global_batch_size=4, n_samples_per_prompt=2, max_tokens_per_gpu=1024, pad_multiple=1,
                      use_rollout_routing_replay=True, loss=LossConfig(), optim=OptimizerConfig(lr=0.0))
    actor = TrainActor(mcfg, cfg, role="actor", seed=0)
    for windowed in (False, True):
        eng = RolloutEngine(mcfg, device="cpu", dtype=torch.float32, num_kv_blocks=128, block_size=8, return_routed_experts=True,
                            windowed_decode=windowed, decode_window=4)
        WeightSync(mcfg, TrainerLayout(), 1, [0], [0]).update_weights(dict(actor.named_local_params()), eng.weights, eng, 1)
        g = torch.Generator().manual_seed(2)
        prompts = [torch.randint(3, 1000, (n,), generator=g).tolist() for n in (7, 7, 9, 9)]
        res = eng.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True), group_keys=[0, 0, 1, 1])
        n_moe = len(eng.weights.moe_layers)
        for r in res:
            assert len(r.routed_experts) == len(r.prompt) + len(r.output) - 1
            assert len(r.routed_experts[0]) == n_moe and len(r.routed_experts[0][0]) == mcfg.moe_top_k
        batch = {"tokens": [r.prompt + r.output for r in res], "response_lengths": [6] * 4, "loss_masks": [[1.0] * 6] * 4,
                 "rewards": [1.0, 0.0, 0.0, 1.0], "rollout_routed_experts": [r.routed_experts for r in res]}
        replayed = []
        orig = RoutingReplay.route.__func__

        def spy(cls, layer, idx):
            out = orig(cls, layer, idx)
            replayed.append((cls.mode, layer, out.clone()))
            return out

        RoutingReplay.route = classmethod(spy)
        try:
            m = actor.train(0, batch)
        finally:
            RoutingReplay.route = classmethod(orig)
        assert RoutingReplay.mode is None and all(mode == "replay" for mode, _, _ in replayed if mode is not None)
        # the first replayed call of the first MoE layer covers all four samples in order: its rows are the engine's ids
        mode, layer, out = next(x for x in replayed if x[0] == "replay")
        m_idx = eng.weights.moe_layers.index(layer)
        want = torch.tensor([pos[m_idx] for pos in res[0].routed_experts])
        assert torch.equal(out[:want.shape[0]], want)
        # same weights, same routing: the engine's log-probs are the trainer's old-policy log-probs
        assert abs(m["ppo_kl"]) < 1e-6


def test_capture_in_a_training_run_and_the_offline_tools(tmp_path, monkeypatch):
    """RELAX_REPLAY_CAPTURE_DIR on a colocated GRPO run: the advantage and loss stages of the chosen rollouts are
    written by the background writer; the bundle validates, replays clean on this host, names the first divergence
    when an implementation changes, and notices a record that was tampered with."""
    import json
    import os

    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller
    from relax_b200.utils import replay as R

    root = tmp_path / "bundles"
    monkeypatch.setenv("RELAX_REPLAY_CAPTURE_DIR", str(root))
    monkeypatch.setenv("RELAX_REPLAY_CAPTURE_ROLLOUTS", "1,2")
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "3", "--rollout-max-response-len", "6", "--lr", "1e-3", "--rm-type", "token_sum_parity",
                    "--use-kl-loss", "--kl-loss-coef", "0.01", "--max-tokens-per-gpu", "4096"])       # one micro-batch per optimizer step
    c = Controller(a, device="cpu")
    for _ in range(3):
        c.runner.step()
    c.runner.actor.replay.close()
    c.runner.close()
    bundle = str(root / "rank-0")
    m = R.load_manifest(bundle)
    assert m["identity"]["model"] == "tiny" and m["identity"]["layout"]["dp"] == [0, 1] and len(m["identity"]["config_sha"]) == 16
    recs = R.select_records(m["records"])
    assert {r["rollout_id"] for r in recs} == {1, 2}                              # rollout 0 was not asked for
    # two optimizer steps of four samples, one micro-batch per sample: one record per micro-batch
    assert [r["stage"] for r in recs if r["rollout_id"] == 1] == ["advantages"] + ["loss"] * 8
    assert [r["step_id"] for r in recs if r["rollout_id"] == 1] == [None] + [0] * 4 + [1] * 4 and all(r["sha256"] for r in recs)
    assert R.validate_bundle(bundle) == [] and R.validate_bundle(str(root)) == []
    assert R.main(["validate", bundle]) == 0 and R.main(["replay", bundle, "--stage", "loss"]) == 0 and R.main(["inspect", str(root)]) == 0
    reps = R.replay_bundle(str(root))
    assert len(reps) == 18 and all(r["ok"] for r in reps) and R.first_divergence(reps) is None
    only = R.replay_bundle(bundle, stages=["loss"], steps=[(2, 1)])
    assert [(r["rollout_id"], r["step_id"]) for r in only] == [(2, 1)] * 4
    # a changed advantage estimator is found at the first record it touches
    fns = R.default_stage_functions()
    good = fns["advantages"]
    fns["advantages"] = lambda **kw: {k: v * 1.001 for k, v in good(**kw).items()}
    first = R.first_divergence(R.replay_bundle(bundle, fns))
    assert first["stage"] == "advantages" and first["rollout_id"] == 1 and first["field"].startswith("out.")
    # integrity: a modified record and a missing COMPLETE marker are reported
    victim = os.path.join(bundle, recs[1]["file"])
    with open(victim, "ab") as f:
        f.write(b"x")
    os.remove(os.path.join(bundle, "COMPLETE"))
    problems = R.validate_bundle(bundle)
    assert any("checksum" in p for p in problems) and any("COMPLETE" in p for p in problems) and R.main(["validate", bundle]) == 1
