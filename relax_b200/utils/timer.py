"""Named wall-clock spans, optional CUDA-event device spans, Chrome-trace export.

Spans become ``perf/<name>_time`` metrics; with a FLOPs estimate they also give
per-GPU TFLOP/s and MFU (counterpart of relax/utils/timer.py and
relax/utils/training/train_metric_utils.py:23-60).
"""
from __future__ import annotations

import contextlib
import json
import os
import threading
import time
from dataclasses import dataclass, field
from typing import Optional


@dataclass
class TimelineEvent:
    name: str
    start_us: float
    dur_us: float
    pid: int = 0
    tid: int = 0
    args: dict = field(default_factory=dict)

    def to_chrome(self):
        return {"name": self.name, "ph": "X", "ts": self.start_us, "dur": self.dur_us, "pid": self.pid,
                "tid": self.tid, "args": self.args}


class Timer:
    def __init__(self, record_timeline: bool = False, pid: int = 0):
        self.totals: dict[str, float] = {}
        self.counts: dict[str, int] = {}
        self.events: list[TimelineEvent] = []
        self.record_timeline = record_timeline
        self.pid = pid
        self._open: dict[str, float] = {}
        self._lock = threading.Lock()
        self._device_spans: list = []

    def start(self, name: str):
        self._open[name] = time.perf_counter()

    def end(self, name: str) -> float:
        t0 = self._open.pop(name)
        dt = time.perf_counter() - t0
        with self._lock:
            self.totals[name] = self.totals.get(name, 0.0) + dt
            self.counts[name] = self.counts.get(name, 0) + 1
            if self.record_timeline:
                self.events.append(TimelineEvent(name, t0 * 1e6, dt * 1e6, self.pid, threading.get_ident() % 1000))
        return dt

    @contextlib.contextmanager
    def span(self, name: str):
        self.start(name)
        try:
            yield
        finally:
            self.end(name)

    @contextlib.contextmanager
    def device_span(self, name: str, stream=None):
        """Time a region with CUDA events on the launching stream; the elapsed
        time is resolved lazily by :meth:`resolve_device_spans` so no
        synchronisation is inserted into the hot path."""
        import torch

        if not torch.cuda.is_available():
            with self.span(name):
                yield
            return
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(stream)
        try:
            yield
        finally:
            e.record(stream)
            self._device_spans.append((name, s, e))

    def resolve_device_spans(self):
        import torch

        if self._device_spans:
            torch.cuda.synchronize()
        for name, s, e in self._device_spans:
            dt = s.elapsed_time(e) / 1e3
            self.totals[name] = self.totals.get(name, 0.0) + dt
            self.counts[name] = self.counts.get(name, 0) + 1
        self._device_spans = []

    def log_dict(self, reset: bool = True, prefix: str = "perf/") -> dict:
        self.resolve_device_spans()
        out = {f"{prefix}{k}_time": v for k, v in self.totals.items()}
        if reset:
            self.totals, self.counts = {}, {}
        return out

    def dump_chrome_trace(self, path: str):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            json.dump({"traceEvents": [e.to_chrome() for e in self.events]}, f)


_GLOBAL: Optional[Timer] = None


def global_timer() -> Timer:
    global _GLOBAL
    if _GLOBAL is None:
        _GLOBAL = Timer()
    return _GLOBAL
