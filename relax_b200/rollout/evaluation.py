"""Evaluation rollouts: generate ``n`` samples for every prompt of one or several held-out sets with their own
sampling settings, score them with the set's reward, and report mean reward, pass@k, response length and
truncation ratio per set.

Covers the reference's evaluation path (relax/engine/rollout/sglang_rollout.py eval_rollout :1142-1296; the eval
flag group of relax/utils/arguments.py :1555 - ``--eval-interval``, ``--eval-prompt-data name path ...``,
``--n-samples-per-eval-prompt``, ``--eval-temperature / top-p / top-k``, ``--eval-max-response-len``; per-dataset
overrides of relax/utils/training/eval_config.py).  Nothing of an evaluation rollout reaches the trainer.
"""
from __future__ import annotations

import json
import math
import statistics
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

from ..types import Sample, SampleStatus


@dataclass
class EvalDataset:
    name: str
    prompts: List[list]                       # token ids per prompt
    labels: List[Any] = field(default_factory=list)
    n_samples_per_prompt: int = 1
    temperature: Optional[float] = None       # None: the run's eval default
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    max_response_len: Optional[int] = None
    rm_type: Optional[str] = None             # None: the run's reward
    metadata: List[dict] = field(default_factory=list)


def pass_at_k(n: int, c: int, k: int) -> float:
    """Unbiased estimate of P(at least one of k samples is correct) from ``c`` correct out of ``n`` drawn:
    ``1 - C(n - c, k) / C(n, k)``."""
    if k > n:
        raise ValueError("k > n")
    if n - c < k:
        return 1.0
    return 1.0 - math.prod((n - c - i) / (n - i) for i in range(k))


def _scalar(r, key: Optional[str] = None) -> float:
    if isinstance(r, dict):
        r = r[key] if key and key in r else r.get("score", r.get("reward", 0.0))
    return float(r)


def summarize(name: str, groups: Sequence[Sequence[Sample]], correct_threshold: float = 0.5,
              reward_key: Optional[str] = None) -> Dict[str, float]:
    """Metrics of one evaluated set; ``groups[i]`` are the samples of prompt ``i``.  ``reward_key`` picks the entry of
    dict-valued rewards (``--eval-reward-key``)."""
    rewards = [_scalar(s.reward, reward_key) for g in groups for s in g]
    lens = [s.response_length for g in groups for s in g]
    trunc = [s.status == SampleStatus.TRUNCATED for g in groups for s in g]
    out = {f"eval/{name}": statistics.fmean(rewards) if rewards else 0.0,
           f"eval/{name}/response_len/mean": statistics.fmean(lens) if lens else 0.0,
           f"eval/{name}/response_len/max": float(max(lens)) if lens else 0.0,
           f"eval/{name}-truncated_ratio": sum(trunc) / max(1, len(trunc)),
           f"eval/{name}/num_prompts": float(len(groups))}
    n = min((len(g) for g in groups), default=0)
    k = 1
    while n >= 1 and k <= n:
        vals = [pass_at_k(len(g), sum(_scalar(s.reward, reward_key) > correct_threshold for s in g), k) for g in groups]
        out[f"eval/{name}-pass@{k}"] = statistics.fmean(vals)
        k *= 2
    return out


def load_eval_datasets(pairs: Sequence[str], tokenize: Callable[[Any], list], input_key: str = "prompt", label_key: str = "label",
                       n_samples_per_prompt: int = 1, size: Optional[int] = None, max_prompt_len: Optional[int] = None,
                       overrides: Optional[Dict[str, dict]] = None) -> List[EvalDataset]:
    """``pairs`` is the flat ``name path name path ...`` list of ``--eval-prompt-data``; rows are JSONL.  ``overrides``
    maps a set name to per-set fields (``n_samples_per_prompt``, ``temperature``, ``max_response_len``, ``rm_type`` ...)."""
    if len(pairs) % 2:
        raise ValueError("--eval-prompt-data takes name/path pairs")
    out = []
    for name, path in zip(pairs[0::2], pairs[1::2]):
        prompts, labels, metas = [], [], []
        with open(path, encoding="utf-8") as f:
            for line in f:
                if not line.strip():
                    continue
                row = json.loads(line)
                toks = tokenize(row[input_key])
                if max_prompt_len and len(toks) > max_prompt_len:
                    continue
                prompts.append(toks)
                labels.append(row.get(label_key))
                metas.append(row.get("metadata") or {})
                if size and len(prompts) >= size:
                    break
        ds = EvalDataset(name, prompts, labels, n_samples_per_prompt, metadata=metas)
        for k, v in (overrides or {}).get(name, {}).items():
            if not hasattr(ds, k):
                raise KeyError(f"unknown eval override {k!r} for set {name!r}")
            setattr(ds, k, v)
        out.append(ds)
    return out


def evaluate(engine, datasets: Sequence[EvalDataset], reward_fn: Callable[[Sample], Any], sampling_defaults,
             decode: Optional[Callable[[list], str]] = None, reward_fns: Optional[Dict[str, Callable]] = None,
             reward_key: Optional[str] = None, generate_fn: Optional[Callable] = None) -> Dict[str, float]:
    """Run every set through ``engine.generate`` (one call per set, all samples batched) and score it.
    ``sampling_defaults`` is a :class:`~relax_b200.rollout.engine.SamplingParams`; per-set fields override it.
    ``generate_fn(engine, samples, sampling_params) -> samples``: the run's custom generate function produces the
    evaluation samples as well (multi-turn environments, agent programs; the reference's ``--eval-function-path``
    defaults to its rollout function); samples it has scored keep their reward."""
    import dataclasses as _dc

    metrics: Dict[str, float] = {}
    for ds in datasets:
        sp = _dc.replace(sampling_defaults,
                         **{k: v for k, v in (("temperature", ds.temperature), ("top_p", ds.top_p), ("top_k", ds.top_k),
                                              ("max_new_tokens", ds.max_response_len)) if v is not None})
        n = ds.n_samples_per_prompt
        flat_prompts = [p for p in ds.prompts for _ in range(n)]
        keys = [i for i in range(len(ds.prompts)) for _ in range(n)]
        score = (reward_fns or {}).get(ds.rm_type, reward_fn) if ds.rm_type else reward_fn
        groups: List[List[Sample]] = [[] for _ in ds.prompts]
        if generate_fn is not None:
            shells = [Sample(group_index=gi, index=j, prompt=(decode(list(p)) if decode is not None else list(p)), tokens=list(p),
                             label=ds.labels[gi] if ds.labels else None, metadata=dict(ds.metadata[gi]) if ds.metadata else {})
                      for j, (gi, p) in enumerate(zip(keys, flat_prompts))]
            fn = getattr(generate_fn, "eval_variant", generate_fn)
            for s in fn(engine, shells, sp):
                if s.remove_sample:
                    continue
                if s.reward is None:
                    s.reward = score(s)
                groups[s.group_index].append(s)
            metrics.update(summarize(ds.name, [g for g in groups if g], reward_key=reward_key))
            continue
        res = engine.generate(flat_prompts, sp, group_keys=keys)
        for gi, r in zip(keys, res):
            s = Sample(group_index=gi, index=len(groups[gi]), prompt=list(r.prompt), tokens=list(r.prompt) + list(r.output),
                       response_length=len(r.output), label=ds.labels[gi] if ds.labels else None,
                       metadata=dict(ds.metadata[gi]) if ds.metadata else {},
                       status=SampleStatus.TRUNCATED if r.finish_reason == "length" else SampleStatus.COMPLETED)
            if decode is not None:
                s.response = decode(list(r.output))
            s.reward = score(s)
            groups[gi].append(s)
        metrics.update(summarize(ds.name, groups, reward_key=reward_key))
    return metrics
