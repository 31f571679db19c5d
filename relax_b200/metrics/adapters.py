"""Tracking adapters behind the metrics service: JSONL file, console, TensorBoard, and the optional
third-party trackers (wandb, clearml, apprise notifications) which are used only when their package
is importable - the reference wires the same four (relax/utils/metrics/adapters, tracking_utils.py).
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Dict, Optional


class JsonlAdapter:
    def __init__(self, path: str):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self.f = open(path, "a", buffering=1)

    def log(self, step: int, rec: Dict[str, float]):
        self.f.write(json.dumps({"step": step, "time": time.time(), **rec}) + "\n")

    def log_error(self, rec: dict):
        self.f.write(json.dumps({"error": rec}) + "\n")

    def close(self):
        self.f.close()


class ConsoleAdapter:
    def __init__(self, keys: Optional[list] = None, stream=None):
        self.keys, self.stream = keys, stream or sys.stderr

    def log(self, step: int, rec: Dict[str, float]):
        items = [(k, rec[k]) for k in (self.keys or sorted(rec)) if k in rec]
        print(f"[step {step}] " + "  ".join(f"{k}={v:.6g}" for k, v in items), file=self.stream, flush=True)


class TensorBoardAdapter:
    def __init__(self, log_dir: str):
        from torch.utils.tensorboard import SummaryWriter  # needs the tensorboard package

        self.w = SummaryWriter(log_dir)

    def log(self, step: int, rec: Dict[str, float]):
        for k, v in rec.items():
            self.w.add_scalar(k, v, step)

    def close(self):
        self.w.close()


class WandbAdapter:
    def __init__(self, project: str, name: Optional[str] = None, config: Optional[dict] = None, mode: str = "offline"):
        import wandb

        self.run = wandb.init(project=project, name=name, config=config or {}, mode=mode)

    def log(self, step: int, rec: Dict[str, float]):
        self.run.log(rec, step=step)

    def close(self):
        self.run.finish()


class ClearMLAdapter:
    def __init__(self, project: str, task_name: str):
        from clearml import Task

        self.task = Task.init(project_name=project, task_name=task_name)
        self.logger = self.task.get_logger()

    def log(self, step: int, rec: Dict[str, float]):
        for k, v in rec.items():
            title, _, series = k.partition("/")
            self.logger.report_scalar(title, series or title, v, step)

    def close(self):
        self.task.close()


class AppriseAdapter:
    """Notifications only (errors and every ``every`` steps a one-line summary)."""

    def __init__(self, urls: list, every: int = 0):
        import apprise

        self.a = apprise.Apprise()
        for u in urls:
            self.a.add(u)
        self.every = every

    def log(self, step: int, rec: Dict[str, float]):
        if self.every and step % self.every == 0:
            self.a.notify(title=f"step {step}", body=", ".join(f"{k}={v:.4g}" for k, v in sorted(rec.items())[:12]))

    def log_error(self, rec: dict):
        self.a.notify(title=f"error in {rec.get('source')}", body=str(rec.get("message"))[:2000])


def build_adapters(args) -> list:
    """Adapters selected by the tracking flags (``--use-tensorboard``, ``--use-wandb``, ...).  A tracker whose
    package is missing is skipped with a warning instead of failing the run."""
    out = []
    out_dir = getattr(args, "metrics_dir", None) or getattr(args, "save", None)
    if out_dir:
        out.append(JsonlAdapter(os.path.join(out_dir, "metrics.jsonl")))

    def _try(make, what):
        try:
            out.append(make())
        except ImportError as e:
            print(f"[metrics] {what} requested but not importable ({e}); skipped", file=sys.stderr)

    if getattr(args, "use_tensorboard", False):
        tb = getattr(args, "tb_dir", None) or os.path.join(out_dir or ".", "tb")
        for part in (getattr(args, "tb_project_name", None), getattr(args, "tb_experiment_name", None)):
            if part:
                tb = os.path.join(tb, str(part))
        _try(lambda: TensorBoardAdapter(tb), "tensorboard")
    if getattr(args, "use_wandb", False):
        _try(lambda: WandbAdapter(getattr(args, "wandb_project", "relax"), getattr(args, "wandb_group", None),
                                  mode=getattr(args, "wandb_mode", "offline")), "wandb")
    if getattr(args, "use_clearml", False):
        _try(lambda: ClearMLAdapter(getattr(args, "clearml_project", "relax"), getattr(args, "clearml_task", "run")), "clearml")
    urls = list(getattr(args, "apprise_urls", None) or []) + list(getattr(args, "notify_urls", None) or [])
    if urls:
        _try(lambda: AppriseAdapter(urls), "apprise")
    if getattr(args, "log_to_console", True):
        out.append(ConsoleAdapter())
    return out
