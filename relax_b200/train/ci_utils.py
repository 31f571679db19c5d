"""Self-checks that a continuous-integration run switches on with ``--ci-test``.

They turn silent training bugs into assertion failures on the first step (what the reference does in
relax/backends/megatron/model.py:1535-1565 and relax/backends/megatron/ci_utils.py):

* on the first optimizer step of a rollout the policy has not moved yet, so the PPO KL between the old and the
  current policy must be (numerically) zero, and on the very first step the KL term to the reference as well;
* gradient norms can be recorded per (role, rollout, step) and compared with a recorded run
  (``--ci-save-grad-norm`` / ``--ci-load-grad-norm``, path templates with ``{role}``, ``{rollout_id}``,
  ``{step_id}``);
* a critic's value head must change after a successful step with a non-zero gradient;
* with MTP-only training only the MTP blocks may receive gradients.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import torch


@dataclass
class CIConfig:
    enabled: bool = False
    save_grad_norm: Optional[str] = None
    load_grad_norm: Optional[str] = None
    disable_kl_checker: bool = False

    @classmethod
    def from_args(cls, a) -> "CIConfig":
        return cls(bool(getattr(a, "ci_test", False)), getattr(a, "ci_save_grad_norm", None),
                   getattr(a, "ci_load_grad_norm", None), bool(getattr(a, "ci_disable_kl_checker", False)))


def check_first_step_kl(ci: CIConfig, metrics: dict, step_id: int, accumulated_step_id: int):
    """``metrics`` are the reduced metrics of one optimizer step (keys as the loss functions name them)."""
    if not ci.enabled or ci.disable_kl_checker:
        return
    get = lambda k: next((float(v) for n, v in metrics.items() if n == k or n.endswith("/" + k)), None)
    ppo_kl, clipfrac, kl_loss = get("ppo_kl"), get("pg_clipfrac"), get("kl_loss")
    if step_id == 0 and ppo_kl is not None and clipfrac is not None:
        assert abs(ppo_kl) < 1e-8, f"first step of a rollout: the policy has not moved, yet ppo_kl = {ppo_kl}: {metrics}"
    if accumulated_step_id == 0 and kl_loss is not None:
        assert kl_loss == 0.0, f"very first step: the policy equals the reference, yet kl_loss = {kl_loss}: {metrics}"


def save_or_check_grad_norm(ci: CIConfig, role: str, rollout_id: int, step_id: int, grad_norm: float, rank: int = 0):
    if ci.save_grad_norm is not None:
        path = ci.save_grad_norm.format(role=role, rollout_id=rollout_id, step_id=step_id)
        if rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            torch.save(float(grad_norm), path)
    elif ci.load_grad_norm is not None:
        path = ci.load_grad_norm.format(role=role, rollout_id=rollout_id, step_id=step_id)
        expected = float(torch.load(path))
        assert math.isclose(float(grad_norm), expected, rel_tol=0.01, abs_tol=0.01), \
            f"grad norm mismatch at {role} rollout {rollout_id} step {step_id}: {grad_norm} != {expected}"


@dataclass
class ValueHeadSnapshot:
    params: list
    has_nonzero_grad: bool


def capture_critic_value_head(model: torch.nn.Module) -> ValueHeadSnapshot:
    snaps, nonzero = [], False
    for name, p in model.named_parameters():
        if "value_head" not in name:
            continue
        g = getattr(p, "main_grad", None)
        g = p.grad if g is None else g
        assert g is not None, f"critic value head parameter {name} has no gradient"
        assert bool(torch.isfinite(g).all()), f"critic value head parameter {name} has a non-finite gradient"
        nonzero = nonzero or bool(torch.count_nonzero(g))
        snaps.append((name, p, p.detach().clone()))
    return ValueHeadSnapshot(snaps, nonzero)


def assert_critic_value_head_updated(snap: ValueHeadSnapshot, update_successful: bool, learning_rates: Sequence[float]):
    if not snap.params or not update_successful or not snap.has_nonzero_grad or not any(lr > 0 for lr in learning_rates):
        return
    assert any(not torch.equal(p.detach(), before) for _, p, before in snap.params), \
        "critic value head did not change after a successful optimizer step with a non-zero gradient"


def check_mtp_only_grad(model: torch.nn.Module, require_non_mtp_zero: bool = True):
    """MTP-only training: the MTP blocks receive gradient, and (optionally) nothing else does."""
    mtp_nonzero = False
    for name, p in model.named_parameters():
        g = getattr(p, "main_grad", None)
        g = p.grad if g is None else g
        if g is None:
            continue
        nz = bool(torch.count_nonzero(g))
        if name.startswith("mtp."):
            mtp_nonzero = mtp_nonzero or nz
        elif require_non_mtp_zero:
            assert not nz, f"non-MTP parameter {name} received a gradient in MTP-only training"
    assert mtp_nonzero, "no MTP parameter received a gradient"
