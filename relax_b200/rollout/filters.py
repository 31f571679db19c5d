"""Dynamic-sampling filters and the over-sampling loop that uses them.

A filter sees one prompt group (the ``n`` samples of a prompt) and says whether it may enter the
training batch; DAPO's filter drops groups whose rewards are all equal (no learning signal under
group-normalised advantages) - relax/engine/filters/__init__.py ``check_reward_nonzero_std``.
The rollout keeps generating ``over_sampling_batch_size`` prompts at a time until
``rollout_batch_size`` groups have passed (relax/engine/rollout/sglang_rollout.py:763-1136);
groups generated beyond the target are handed back to the data source's buffer.
"""
from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence


@dataclass
class FilterOutput:
    keep: bool
    reason: Optional[str] = None


def check_reward_nonzero_std(group: Sequence) -> FilterOutput:
    rewards = [float(s.reward if not isinstance(s.reward, dict) else s.reward.get("score", 0.0)) for s in group]
    mean = sum(rewards) / max(1, len(rewards))
    var = sum((r - mean) ** 2 for r in rewards) / max(1, len(rewards))
    return FilterOutput(var > 1e-12, None if var > 1e-12 else f"zero_std_{round(mean, 4)}")


def load_filter(path: Optional[str]) -> Optional[Callable]:
    """``module.sub:function`` or ``module.sub.function`` -> callable; None passes through."""
    if not path:
        return None
    mod, _, fn = path.replace(":", ".").rpartition(".")
    return getattr(importlib.import_module(mod), fn)


def dynamic_sampling(generate_groups: Callable[[int], List[list]], batch_size: int, over_sampling_batch_size: Optional[int] = None,
                     group_filter: Optional[Callable] = None, max_rounds: int = 64, give_back: Optional[Callable] = None):
    """Collect ``batch_size`` groups that pass ``group_filter``.  Returns ``(groups, stats)``; ``stats`` counts
    the drops per reason.  Surplus passing groups of the last round go to ``give_back`` (the rollout buffer)."""
    over = max(batch_size, over_sampling_batch_size or batch_size)
    kept: List[list] = []
    stats = {"generated_groups": 0, "dropped_groups": 0, "rounds": 0}
    while len(kept) < batch_size:
        if stats["rounds"] >= max_rounds:
            raise RuntimeError(f"dynamic sampling: only {len(kept)}/{batch_size} groups passed after {max_rounds} rounds")
        stats["rounds"] += 1
        want = over if group_filter is not None else batch_size - len(kept)
        groups = generate_groups(want)
        stats["generated_groups"] += len(groups)
        for g in groups:
            out = group_filter(g) if group_filter is not None else FilterOutput(True)
            keep = out.keep if isinstance(out, FilterOutput) else bool(out)
            if keep:
                kept.append(g)
            else:
                stats["dropped_groups"] += 1
                r = getattr(out, "reason", None)
                if r:
                    stats[f"drop/{r}"] = stats.get(f"drop/{r}", 0) + 1
    surplus = kept[batch_size:]
    if surplus and give_back is not None:
        give_back(surplus)
    return kept[:batch_size], stats
