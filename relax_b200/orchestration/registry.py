"""Roles, the role set each execution mode runs, and the algorithm table.

Behavioural counterpart of relax/core/registry.py:23-179.  A *role* here is a
coroutine/thread bound to a subset of ranks of the SPMD job rather than a Ray
Serve deployment.
"""
from __future__ import annotations

import enum
from typing import Iterable


class Role(str, enum.Enum):
    actor = "actor"
    critic = "critic"
    rollout = "rollout"
    advantages = "advantages"
    reference = "reference"
    actor_fwd = "actor_fwd"
    sft = "sft"
    genrm = "genrm"


ROLES_TRAIN_ONLY = (Role.actor,)
ROLES_ROLLOUT_ONLY = (Role.rollout,)
ROLES_COLOCATE = (Role.actor, Role.critic, Role.rollout)
ROLES_SFT_ONLY = (Role.sft, Role.actor)
ROLES_FULLY_ASYNC = (Role.actor, Role.critic, Role.rollout, Role.advantages, Role.reference, Role.actor_fwd)
ROLES_FULLY_ASYNC_ON_POLICY = (Role.actor, Role.critic, Role.rollout, Role.advantages, Role.reference)

# estimator -> (loss kind, needs critic, group baseline)
ALGOS = {
    "grpo": ("policy_loss", False, True),
    "gspo": ("policy_loss", False, True),
    "sapo": ("policy_loss", False, True),
    "cispo": ("policy_loss", False, True),
    "m2po": ("policy_loss", False, True),
    "rloo": ("policy_loss", False, True),
    "reinforce_plus_plus": ("policy_loss", False, False),
    "reinforce_plus_plus_baseline": ("policy_loss", False, True),
    "ppo": ("policy_loss", True, False),
    "on_policy_distillation": ("policy_loss", False, False),
    "sft": ("sft_loss", False, False),
}


def process_role(config) -> tuple:
    """Role set of a run.  The critic is kept only when the estimator needs one."""
    if getattr(config, "debug_rollout_only", False):
        return ROLES_ROLLOUT_ONLY
    if getattr(config, "debug_train_only", False):
        return ROLES_TRAIN_ONLY
    if getattr(config, "loss_type", None) in ("sft", "sft_loss"):
        return ROLES_SFT_ONLY
    est = getattr(config, "advantage_estimator", "grpo")
    needs_critic = ALGOS.get(est, ("policy_loss", False, False))[1]

    def keep(roles: Iterable[Role]) -> tuple:
        return tuple(r for r in roles if r != Role.critic or needs_critic)

    if est == "ppo":
        if config.fully_async:
            return ROLES_FULLY_ASYNC_ON_POLICY if getattr(config, "true_on_policy_mode", False) else ROLES_FULLY_ASYNC
        return ROLES_COLOCATE
    if getattr(config, "hybrid", False):
        return keep(ROLES_COLOCATE)      # ref / actor_fwd run inside the actor by switching weight tags
    if getattr(config, "fully_async", False):
        if getattr(config, "true_on_policy_mode", False):
            return keep(ROLES_FULLY_ASYNC_ON_POLICY)
        return keep(ROLES_FULLY_ASYNC)
    return keep(ROLES_COLOCATE)


def register_extra_roles(roles: tuple, config) -> tuple:
    """Optional roles (relax/core/optional_roles.py): generative reward model, SFT data producer."""
    out = list(roles)
    if getattr(config, "genrm_model_path", None) and Role.genrm not in out:
        out.append(Role.genrm)
    return tuple(out)


def satisfy_staleness(partition_list, current_rollout_id: int, max_staleness: int) -> bool:
    """Rollout ``current_rollout_id + 1`` may start iff it is at most ``max_staleness`` ahead of
    the oldest partition the trainer has not consumed (relax/components/rollout.py:298-315)."""
    if not partition_list:
        return True
    oldest = min(int(p.rsplit("_", 1)[1]) for p in partition_list)
    return current_rollout_id + 1 - oldest <= max_staleness


def assign_ranks(resource: dict, world: int, colocate: bool) -> dict:
    """Map ``--resource`` to rank lists.  Colocated roles share the same ranks; otherwise roles get
    disjoint consecutive blocks in declaration order (the order placement groups are packed in)."""
    out, cursor = {}, 0
    for role, (_serves, gpus) in resource.items():
        if gpus == 0:
            out[role] = ()
            continue
        if colocate and role in ("actor", "rollout", "critic", "reference", "actor_fwd"):
            out[role] = tuple(range(min(gpus, world)))
            continue
        if cursor + gpus > world:
            raise ValueError(f"--resource needs more than the {world} GPUs of this job")
        out[role] = tuple(range(cursor, cursor + gpus))
        cursor += gpus
    return out
