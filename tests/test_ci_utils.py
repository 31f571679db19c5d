"""--ci-test self-checks: first-step KL must vanish, grad norms can be recorded and compared, value head must move."""
import os

import pytest
import torch

from relax_b200.train import ci_utils as CI


def test_first_step_kl_checks():
    ci = CI.CIConfig(enabled=True)
    CI.check_first_step_kl(ci, {"ppo_kl": 0.0, "pg_clipfrac": 0.0, "kl_loss": 0.0}, 0, 0)
    with pytest.raises(AssertionError):
        CI.check_first_step_kl(ci, {"ppo_kl": 1e-3, "pg_clipfrac": 0.0}, 0, 5)
    CI.check_first_step_kl(ci, {"ppo_kl": 1e-3, "pg_clipfrac": 0.0}, 1, 5)          # later steps of a rollout may move
    with pytest.raises(AssertionError):
        CI.check_first_step_kl(ci, {"kl_loss": 1e-4}, 0, 0)
    CI.check_first_step_kl(CI.CIConfig(enabled=True, disable_kl_checker=True), {"ppo_kl": 1.0, "pg_clipfrac": 0.0}, 0, 0)


def test_grad_norm_record_and_compare(tmp_path):
    tmpl = str(tmp_path / "gn" / "{role}_{rollout_id}_{step_id}.pt")
    CI.save_or_check_grad_norm(CI.CIConfig(save_grad_norm=tmpl), "actor", 3, 1, 0.75)
    assert os.path.exists(tmpl.format(role="actor", rollout_id=3, step_id=1))
    CI.save_or_check_grad_norm(CI.CIConfig(load_grad_norm=tmpl), "actor", 3, 1, 0.752)
    with pytest.raises(AssertionError):
        CI.save_or_check_grad_norm(CI.CIConfig(load_grad_norm=tmpl), "actor", 3, 1, 0.9)


def test_trainer_runs_the_checks_and_a_recorded_run_reproduces(tmp_path):
    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.train.actor import TrainActor, TrainConfig

    tmpl = str(tmp_path / "{role}_{rollout_id}_{step_id}.pt")

    def run(ci):
        actor = TrainActor(get_config("tiny"), TrainConfig(pad_multiple=1, global_batch_size=4, n_samples_per_prompt=2, ci=ci,
                                                           loss=LossConfig(use_kl_loss=True, kl_loss_coef=0.01)), seed=3,
                           with_reference=True)
        g = torch.Generator().manual_seed(0)
        toks = [torch.randint(0, 1000, (20,), generator=g).tolist() for _ in range(4)]
        batch = {"tokens": toks, "response_lengths": [8] * 4, "loss_masks": [[1.0] * 8] * 4, "rewards": [1.0, -1.0, 0.5, -0.5]}
        return actor.train(0, batch)["grad_norm"]

    n0 = run(CI.CIConfig(enabled=True, save_grad_norm=tmpl))
    assert os.path.exists(tmpl.format(role="actor", rollout_id=0, step_id=0))
    assert abs(run(CI.CIConfig(enabled=True, load_grad_norm=tmpl)) - n0) < 1e-6


def test_value_head_and_mtp_checks():
    lin = torch.nn.Module()
    lin.value_head = torch.nn.Linear(4, 1, bias=False)
    lin.value_head.weight.grad = torch.ones(1, 4)
    snap = CI.capture_critic_value_head(lin)
    with pytest.raises(AssertionError):
        CI.assert_critic_value_head_updated(snap, True, [1e-3])
    with torch.no_grad():
        lin.value_head.weight.add_(1.0)
    CI.assert_critic_value_head_updated(snap, True, [1e-3])
    m = torch.nn.Module()
    m.mtp = torch.nn.Linear(2, 2)
    m.trunk = torch.nn.Linear(2, 2)
    m.mtp.weight.grad = torch.ones(2, 2)
    m.trunk.weight.grad = torch.zeros(2, 2)
    CI.check_mtp_only_grad(m)
    m.trunk.weight.grad = torch.ones(2, 2)
    with pytest.raises(AssertionError):
        CI.check_mtp_only_grad(m)
