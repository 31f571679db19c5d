"""End-to-end colocated GRPO on CPU/gloo world_size=2: tiny Qwen-style decoder
(2 layers, hidden 256, 4 q / 2 kv heads, head_dim 64, FFN 688, vocab 1024, fp32),
8 prompts x 64 tokens, group size 4, responses up to 64 tokens, temperature 1,
parity reward, GRPO clip 0.2, KL coef 0.001 to a frozen reference, Adam lr 1e-5,
3 steps with a weight sync after each."""
import math

import torch

from tests._mp import run_distributed


def _make_cfg(trainer_tp=1, rollout_tp=1):
    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.orchestration.colocate import ColocateConfig
    from relax_b200.train.actor import TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    return ColocateConfig(
        model=get_config("tiny"),
        train=TrainConfig(advantage_estimator="grpo", n_samples_per_prompt=4, global_batch_size=32,
                          max_tokens_per_gpu=2048,
                          loss=LossConfig(eps_clip=0.2, use_kl_loss=True, kl_loss_coef=0.001, kl_loss_type="k1"),
                          optim=OptimizerConfig(lr=1e-5, clip_grad=1.0)),
        trainer_tp=trainer_tp, rollout_tp=rollout_tp, rollout_batch_size=8, prompt_len=64, max_response_len=64,
        temperature=1.0, rm_type="parity", eos_token_id=3, seed=0, rollout_seed=42)


def _worker(rank, world, trainer_tp, rollout_tp):
    from relax_b200.orchestration.colocate import ColocatedGRPO

    torch.manual_seed(0)
    run = ColocatedGRPO(_make_cfg(trainer_tp, rollout_tp))
    w0 = run.engine.weights.flat.clone()
    hist = []
    for _ in range(3):
        m = run.step()
        hist.append(m)
        # the rollout copy must equal the trainer's weights after each sync
        p = dict(run.actor.named_local_params())
        if trainer_tp == rollout_tp == 1:
            assert torch.equal(run.engine.weights.p["layers.0.o"], p["decoder.layers.0.self_attention.linear_proj.weight"])
    assert run.engine.weight_version == 3
    assert not torch.equal(w0, run.engine.weights.flat)          # training moved the policy
    for m in hist:
        assert math.isfinite(m["loss"]) and math.isfinite(m["grad_norm"]) and m["grad_norm"] > 0
        assert m["train_rollout_logprob_abs_diff"] < 1e-4          # rollout and trainer agree on log-probs
        assert abs(m["ppo_kl"]) < 1e-6 and m["pg_clipfrac"] == 0.0   # first pass over fresh data is on-policy
    assert abs(hist[0]["kl_loss"]) < 1e-7                          # reference == actor before any update
    return [(m["loss"], m["grad_norm"], m["entropy_loss"], m["response_tokens_local"]) for m in hist]


def test_grpo_dp2_three_steps_deterministic():
    a = run_distributed(_worker, 2, 1, 1)
    b = run_distributed(_worker, 2, 1, 1)
    assert a == b                                                   # bitwise repeatable
    # ranks share reduced metrics (loss, grad norm) but generated different responses
    assert [x[:2] for x in a[0]] == [x[:2] for x in a[1]]


def test_grpo_tp2_trainer_and_tp2_rollout():
    out = run_distributed(_worker, 2, 2, 2)
    assert out[0] == out[1]                                         # one engine, one replica: identical views


def _pp_worker(rank, world):
    """Colocated GRPO with a pipeline-parallel trainer (pp = 2): each rank is one stage of the trainer and a whole
    rollout engine, so every weight sync pulls the other stage's layers from the other process."""
    import dataclasses

    from relax_b200.orchestration.colocate import ColocatedGRPO

    cfg = dataclasses.replace(_make_cfg(1, 1), trainer_pp=2)
    run = ColocatedGRPO(cfg)
    assert run.ps.pp.size == 2 and len(run.actor.model.decoder.layers) == 1
    hist = [run.step() for _ in range(2)]
    for m in hist:
        assert math.isfinite(m["loss"]) and m["grad_norm"] > 0
        assert m["train_rollout_logprob_abs_diff"] < 1e-4        # the engine really holds all layers of the new policy
    assert run.engine.weight_version == 2
    return [(m["loss"], m["grad_norm"]) for m in hist], run.engine.weights.flat.double().sum().item()


def test_grpo_pipeline_parallel_trainer_two_stages():
    out = run_distributed(_pp_worker, 2, timeout=600)
    assert out[0][0] == out[1][0]                 # both stages report the same loss / grad norm
    assert abs(out[0][1] - out[1][1]) < 1e-6      # both engines hold the same full set of weights


def _ep_worker(rank, world):
    """Colocated GRPO of a mixture-of-experts model with expert parallelism on both sides: trainer TP1 x EP2 (the two
    ranks are also the two data-parallel replicas), one engine of EP2 on the same ranks."""
    import dataclasses

    from relax_b200.models.config import get_config
    from relax_b200.orchestration.colocate import ColocatedGRPO

    cfg = dataclasses.replace(_make_cfg(1, 1), model=get_config("tiny-moe"), trainer_ep=2, rollout_ep=2)
    run = ColocatedGRPO(cfg)
    assert run.ps.ep.size == 2 and run.engine.ep is not None and run.num_engines == 1
    assert run.engine.weights.p["layers.0.experts_gate_up"].shape[0] == cfg.model.num_experts // 2
    hist = [run.step() for _ in range(2)]
    for m in hist:
        assert math.isfinite(m["loss"]) and m["grad_norm"] > 0
        assert m["train_rollout_logprob_abs_diff"] < 1e-4      # the EP engine computes what the EP trainer computes
    return [(m["loss"], m["grad_norm"]) for m in hist]


def test_grpo_expert_parallel_trainer_and_engine():
    out = run_distributed(_ep_worker, 2, timeout=600)
    assert out[0] == out[1]


def _cp_worker(rank, world):
    """Colocated GRPO with a context-parallel trainer (cp = 2): the two ranks are ONE trainer replica (each holds a
    slice of every sequence) and two engines, so every rank must train on the rows of both engines."""
    import dataclasses

    from relax_b200.orchestration.colocate import ColocatedGRPO

    cfg = dataclasses.replace(_make_cfg(1, 1), trainer_cp=2)
    run = ColocatedGRPO(cfg)
    assert run.ps.cp.size == 2 and run.ps.dp.size == 1 and run.num_engines == 2
    hist = [run.step() for _ in range(2)]
    for m in hist:
        assert math.isfinite(m["loss"]) and m["grad_norm"] > 0
        assert m["train_rollout_logprob_abs_diff"] < 1e-4      # both ranks score the same rows the engines produced
    return [(m["loss"], m["grad_norm"]) for m in hist], run.engine.weights.flat.double().sum().item()


def test_grpo_context_parallel_trainer():
    out = run_distributed(_cp_worker, 2, timeout=600)
    assert out[0][0] == out[1][0]                 # one replica: both ranks report the same loss / grad norm
    assert abs(out[0][1] - out[1][1]) < 1e-6
