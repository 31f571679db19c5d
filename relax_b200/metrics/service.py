"""Metrics service: every role reports scalars against a training step; the service merges them,
flushes a step once it is reported complete (or when a later step starts) and fans the record out
to tracking adapters.  It runs in-process (``MetricsService``) and optionally behind a small HTTP
endpoint (``serve``) with the reference's routes ``/log_metric /log_metrics_batch /report_step
/log_error /health`` (relax/utils/metrics/service.py), for roles that live in other processes;
``MetricsClient`` speaks to either.
"""
from __future__ import annotations

import json
import threading
import time
import urllib.request
from collections import defaultdict
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, Iterable, List, Optional


class MetricsService:
    def __init__(self, adapters: Iterable = (), keep_last: int = 512):
        self.adapters = list(adapters)
        self._lock = threading.Lock()
        self._pending: Dict[int, Dict[str, float]] = defaultdict(dict)
        self._counts: Dict[int, Dict[str, int]] = defaultdict(dict)
        self._flushed: List[tuple] = []
        self._errors: List[dict] = []
        self._keep = keep_last
        self._max_flushed_step = -1

    # -- reporting
    def log_metric(self, step: int, name: str, value: float, reduce: str = "last"):
        """``reduce``: how repeated reports of one metric inside a step combine (last / mean / sum / max / min)."""
        with self._lock:
            cur, cnt = self._pending[step], self._counts[step]
            v = float(value)
            if name not in cur or reduce == "last":
                cur[name], cnt[name] = v, 1
            elif reduce == "sum":
                cur[name] += v
            elif reduce == "max":
                cur[name] = max(cur[name], v)
            elif reduce == "min":
                cur[name] = min(cur[name], v)
            elif reduce == "mean":
                n = cnt[name]
                cur[name] = (cur[name] * n + v) / (n + 1)
                cnt[name] = n + 1
            else:
                raise ValueError(f"unknown reduce {reduce!r}")

    def log_metrics_batch(self, step: int, metrics: Dict[str, float], reduce: str = "last"):
        for k, v in metrics.items():
            self.log_metric(step, k, v, reduce)

    def report_step(self, step: int):
        """Step ``step`` (and every earlier one still pending) is complete: flush in order."""
        with self._lock:
            ready = sorted(s for s in self._pending if s <= step)
            recs = [(s, self._pending.pop(s)) for s in ready]
            for s in ready:
                self._counts.pop(s, None)
        for s, rec in recs:
            self._emit(s, rec)

    def log_error(self, source: str, message: str, step: Optional[int] = None):
        rec = {"time": time.time(), "source": source, "message": message, "step": step}
        with self._lock:
            self._errors.append(rec)
            self._errors = self._errors[-self._keep:]
        for a in self.adapters:
            if hasattr(a, "log_error"):
                a.log_error(rec)

    # -- queries
    def history(self) -> List[tuple]:
        with self._lock:
            return list(self._flushed)

    def errors(self) -> List[dict]:
        with self._lock:
            return list(self._errors)

    def _emit(self, step: int, rec: Dict[str, float]):
        with self._lock:
            self._flushed.append((step, dict(rec)))
            self._flushed = self._flushed[-self._keep:]
            self._max_flushed_step = max(self._max_flushed_step, step)
        for a in self.adapters:
            a.log(step, rec)

    def close(self):
        with self._lock:
            last = max(self._pending) if self._pending else None
        if last is not None:
            self.report_step(last)
        for a in self.adapters:
            if hasattr(a, "close"):
                a.close()


class _Handler(BaseHTTPRequestHandler):
    service: MetricsService = None

    def log_message(self, *a):  # silence the default stderr access log
        pass

    def _reply(self, code: int, body: dict):
        data = json.dumps(body).encode()
        self.send_response(code)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(data)))
        self.end_headers()
        self.wfile.write(data)

    def do_GET(self):
        if self.path == "/health":
            return self._reply(200, {"status": "ok"})
        if self.path == "/history":
            return self._reply(200, {"history": self.service.history()})
        self._reply(404, {"error": "unknown route"})

    def do_POST(self):
        n = int(self.headers.get("Content-Length", "0"))
        try:
            body = json.loads(self.rfile.read(n) or b"{}")
            svc = self.service
            if self.path == "/log_metric":
                svc.log_metric(int(body["step"]), body["name"], body["value"], body.get("reduce", "last"))
            elif self.path == "/log_metrics_batch":
                svc.log_metrics_batch(int(body["step"]), body["metrics"], body.get("reduce", "last"))
            elif self.path == "/report_step":
                svc.report_step(int(body["step"]))
            elif self.path == "/log_error":
                svc.log_error(body.get("source", "?"), body.get("message", ""), body.get("step"))
            else:
                return self._reply(404, {"error": "unknown route"})
            self._reply(200, {"ok": True})
        except Exception as e:  # noqa: BLE001
            self._reply(400, {"error": f"{type(e).__name__}: {e}"})


def serve(service: MetricsService, host: str = "127.0.0.1", port: int = 0):
    """Start the HTTP front of ``service`` on a daemon thread; returns ``(server, url)``."""
    handler = type("Handler", (_Handler,), {"service": service})
    srv = ThreadingHTTPServer((host, port), handler)
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    return srv, f"http://{host}:{srv.server_address[1]}"


class MetricsClient:
    """Same calls as :class:`MetricsService`, in-process (``service=``) or over HTTP (``url=``)."""

    def __init__(self, service: Optional[MetricsService] = None, url: Optional[str] = None, timeout: float = 5.0):
        assert (service is None) != (url is None), "give exactly one of service / url"
        self.service, self.url, self.timeout = service, url, timeout

    def _post(self, route: str, body: dict):
        req = urllib.request.Request(self.url + route, data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=self.timeout) as r:
            return json.loads(r.read())

    def log_metric(self, step, name, value, reduce="last"):
        if self.service:
            return self.service.log_metric(step, name, value, reduce)
        self._post("/log_metric", {"step": step, "name": name, "value": float(value), "reduce": reduce})

    def log_metrics_batch(self, step, metrics, reduce="last"):
        if self.service:
            return self.service.log_metrics_batch(step, metrics, reduce)
        self._post("/log_metrics_batch", {"step": step, "metrics": {k: float(v) for k, v in metrics.items()}, "reduce": reduce})

    def report_step(self, step):
        if self.service:
            return self.service.report_step(step)
        self._post("/report_step", {"step": step})

    def log_error(self, source, message, step=None):
        if self.service:
            return self.service.log_error(source, message, step)
        self._post("/log_error", {"source": source, "message": message, "step": step})
