"""Trajectory replay: record the exact inputs and outputs of the numerically delicate stages of a
training step (reward post-processing, advantage estimation, the policy loss) and re-run them
offline, to bisect a regression or reproduce a divergence without the cluster
(relax/utils/replay/: capture hooks in the loss / advantage / reward stages, bundle, offline runner).

A bundle is a directory: ``manifest.json`` lists the captured records; each record is one ``.pt``
file holding ``{"inputs": {...}, "outputs": {...}}`` with tensors moved to the CPU.
"""
from __future__ import annotations

import dataclasses
import json
import os
import time
from typing import Callable, Dict, Iterable, Optional

import torch

STAGES = ("reward", "advantages", "loss")


def _to_cpu(x):
    if torch.is_tensor(x):
        return x.detach().cpu()
    if dataclasses.is_dataclass(x) and not isinstance(x, type):
        return {"__dataclass__": type(x).__module__ + ":" + type(x).__qualname__,
                "fields": {f.name: _to_cpu(getattr(x, f.name)) for f in dataclasses.fields(x)}}
    if isinstance(x, dict):
        return {k: _to_cpu(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_to_cpu(v) for v in x)
    return x


def _restore(x):
    if isinstance(x, dict) and "__dataclass__" in x:
        import importlib

        mod, _, qual = x["__dataclass__"].partition(":")
        cls = importlib.import_module(mod)
        for part in qual.split("."):
            cls = getattr(cls, part)
        return cls(**{k: _restore(v) for k, v in x["fields"].items()})
    if isinstance(x, dict):
        return {k: _restore(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_restore(v) for v in x)
    return x


class ReplayRecorder:
    def __init__(self, out_dir: Optional[str], stages: Iterable[str] = STAGES, max_records: int = 64, rank: int = 0):
        self.out_dir, self.stages, self.max_records, self.rank = out_dir, set(stages), max_records, rank
        self.records: list = []
        if out_dir:
            os.makedirs(out_dir, exist_ok=True)

    @property
    def enabled(self) -> bool:
        return self.out_dir is not None

    def capture(self, stage: str, rollout_id: int, inputs: dict, outputs) -> Optional[str]:
        if not self.enabled or stage not in self.stages or len(self.records) >= self.max_records:
            return None
        name = f"{stage}_r{rollout_id}_rank{self.rank}_{len(self.records):04d}.pt"
        torch.save({"inputs": _to_cpu(inputs), "outputs": _to_cpu(outputs)}, os.path.join(self.out_dir, name))
        self.records.append({"stage": stage, "rollout_id": rollout_id, "file": name, "time": time.time()})
        with open(os.path.join(self.out_dir, "manifest.json"), "w") as f:
            json.dump({"records": self.records}, f, indent=1)
        return name

    def wrap(self, stage: str, fn: Callable, rollout_id_fn: Callable[[], int] = lambda: -1) -> Callable:
        """``fn(**kwargs)`` recorded transparently."""
        def inner(**kw):
            out = fn(**kw)
            self.capture(stage, rollout_id_fn(), kw, out)
            return out

        return inner


def _compare(a, b, atol, rtol, path, diffs):
    if torch.is_tensor(a) and torch.is_tensor(b):
        if a.shape != b.shape:
            diffs.append((path, f"shape {tuple(a.shape)} vs {tuple(b.shape)}"))
        elif not torch.allclose(a.float(), b.float(), atol=atol, rtol=rtol, equal_nan=True):
            diffs.append((path, f"max abs diff {float((a.float() - b.float()).abs().max()):.3e}"))
    elif isinstance(a, dict) and isinstance(b, dict):
        for k in a:
            if k in b:
                _compare(a[k], b[k], atol, rtol, f"{path}.{k}", diffs)
            else:
                diffs.append((f"{path}.{k}", "missing in replay"))
    elif isinstance(a, (list, tuple)) and isinstance(b, (list, tuple)):
        if len(a) != len(b):
            diffs.append((path, f"length {len(a)} vs {len(b)}"))
        for i, (x, y) in enumerate(zip(a, b)):
            _compare(x, y, atol, rtol, f"{path}[{i}]", diffs)
    elif isinstance(a, float) and isinstance(b, float):
        if abs(a - b) > atol + rtol * abs(a):
            diffs.append((path, f"{a} vs {b}"))


def default_stage_functions() -> Dict[str, Callable]:
    from ..algo import loss as L
    from ..algo.ppo_utils import post_process_rewards

    def run_loss(log_probs, entropy, batch, cfg):
        loss, metrics = L.policy_loss(log_probs, entropy, batch, cfg)
        return {"loss": loss, "metrics": metrics}

    def run_adv(**kw):
        adv, ret = L.compute_advantages_and_returns(**kw)
        return {"advantages": adv, "returns": ret}

    return {"loss": run_loss, "advantages": run_adv, "reward": lambda **kw: post_process_rewards(**kw)}


def replay_bundle(bundle_dir: str, stage_fns: Optional[Dict[str, Callable]] = None, atol: float = 1e-6,
                  rtol: float = 1e-5) -> list:
    """Re-run every record of a bundle through ``stage_fns[stage](**inputs)``; returns one report per record:
    ``{"file", "stage", "ok", "diffs": [(where, what), ...]}``."""
    fns = stage_fns or default_stage_functions()
    manifest = json.load(open(os.path.join(bundle_dir, "manifest.json")))
    reports = []
    for rec in manifest["records"]:
        blob = torch.load(os.path.join(bundle_dir, rec["file"]), weights_only=False)
        fn = fns.get(rec["stage"])
        if fn is None:
            reports.append({"file": rec["file"], "stage": rec["stage"], "ok": None, "diffs": [("", "no function for this stage")]})
            continue
        out = _to_cpu(fn(**_restore(blob["inputs"])))
        diffs: list = []
        _compare(blob["outputs"], out, atol, rtol, "out", diffs)
        reports.append({"file": rec["file"], "stage": rec["stage"], "ok": not diffs, "diffs": diffs})
    return reports


def main(argv=None):
    import argparse

    ap = argparse.ArgumentParser(description="Re-run a replay bundle and report where the results differ")
    ap.add_argument("bundle")
    ap.add_argument("--atol", type=float, default=1e-6)
    ap.add_argument("--rtol", type=float, default=1e-5)
    a = ap.parse_args(argv)
    reps = replay_bundle(a.bundle, atol=a.atol, rtol=a.rtol)
    for r in reps:
        print(("OK   " if r["ok"] else "DIFF ") + r["file"] + "".join(f"\n      {w}: {d}" for w, d in r["diffs"]))
    return 0 if all(r["ok"] for r in reps) else 1


if __name__ == "__main__":
    raise SystemExit(main())
