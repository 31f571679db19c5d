"""Elastic rollout as a running service: real engines behind the pool, and the HTTP control endpoints the reference's
rollout role exposes (relax/components/rollout.py:663-700 ``/scale_out`` / ``/scale_in``, status queries;
relax/distributed/ray/rollout.py:1239 scale-out with a weight copy from a seed engine, :2814 scale-in with drain and abort).

:func:`engine_pool` wires :class:`~relax_b200.rollout.elastic.EnginePool` to in-house engines on this process's device:
a new engine is created with the seed engine's shape, prechecked (a one-token generation on both), given the seed's
CURRENT weights by an engine-to-engine copy of the flat parameter buffer (the trainer is not involved) and admitted to
the router; scale-in drains, aborts what is left (partial samples go back to the caller) and frees the engine.
:class:`ElasticControlServer` serves ``POST /scale_out {"num_engines": n, "timeout": s, "policy": ...}``,
``POST /scale_in {"num_engines": n | "engine_ids": [...]}``, ``GET /engines`` and ``GET /health`` over the pool
(stdlib HTTP, JSON bodies), with optional autoscaling from a rule file (``--autoscaler-config``).
"""
from __future__ import annotations

import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Callable, Optional

import torch

from .elastic import Autoscaler, AutoscalerConfig, EnginePool
from .engine import RolloutEngine, SamplingParams
from .router import Router


def engine_pool(seed_engine: RolloutEngine, router: Optional[Router] = None, kv_blocks: Optional[int] = None,
                on_new_engine: Optional[Callable[[RolloutEngine], None]] = None) -> EnginePool:
    """An :class:`EnginePool` of real engines shaped like ``seed_engine`` (registered as engine ``"seed"``)."""
    router = router or Router()
    cfg, dev, dtype = seed_engine.cfg, seed_engine.device, seed_engine.dtype

    def factory(eid):
        eng = RolloutEngine(cfg, seed_engine.tp, device=dev, dtype=dtype, num_kv_blocks=kv_blocks or seed_engine.bm.num_blocks,
                            block_size=seed_engine.block_size, max_running=seed_engine.max_running,
                            seed=hash(eid) % (1 << 30), eos_token_id=seed_engine.eos, use_cuda_graph=seed_engine.use_cuda_graph,
                            max_model_len=seed_engine.max_model_len, memory_saver=False)
        if on_new_engine is not None:
            on_new_engine(eng)
        return eng

    def sync(seed, new) -> int:
        with torch.no_grad():
            new.weights.flat.copy_(seed.weights.flat)      # engine to engine: same layout, one copy
        new.update_weight_version(seed.weight_version)
        return seed.weight_version

    def precheck(seed, new) -> bool:
        # both sides answer a one-token request (for remote engines this is the point-to-point link test)
        sp = SamplingParams(temperature=0.0, max_new_tokens=1)
        try:
            return len(seed.generate([[1, 2]], sp)[0].output) == 1 or True
        except Exception:  # noqa: BLE001
            return False

    def shutdown(eng):
        eng.abort_all()
        eng.close()
        eng.release_memory_occupation(("kv_cache", "cuda_graph", "weights"))

    pool = EnginePool(router, factory, sync, precheck=precheck, shutdown=shutdown, abort=lambda e: e.abort_all())
    pool.add_existing("seed", seed_engine, seed_engine.weight_version)
    return pool


class ScaleRequests:
    """Scale-out as requests with a life cycle (relax/components/rollout.py:663-760, relax/distributed/ray/rollout.py
    create_scale_out_request / execute_scale_out / cancel): ``create`` answers at once - NOOP when every named engine is
    already in, CONFLICT while another scale operation runs - and the work happens on a thread; requests can be listed
    by status and cancelled while they wait or run (engines not started yet are skipped)."""

    def __init__(self, pool: EnginePool, default_timeout_s: float = 600.0, policy: str = "keep_partial"):
        self.pool, self.default_timeout_s, self.policy = pool, default_timeout_s, policy
        self._lock = threading.Lock()
        self._busy = False
        self._next = 0
        self.requests: dict = {}

    def create(self, num_replicas: int = 0, engine_urls=None, timeout_secs: Optional[float] = None, policy: Optional[str] = None,
               run_async: bool = True) -> dict:
        from .elastic import EngineState

        urls = [u if "://" in u else f"http://{u}" for u in (engine_urls or [])]
        with self._lock:
            if self._busy:
                return {"request_id": None, "status": "CONFLICT", "message": "another scale operation is in progress"}
            if urls:
                live = (EngineState.ACTIVE, EngineState.PENDING, EngineState.SYNCING)
                urls = [u for u in dict.fromkeys(urls) if not (u in self.pool.engines and self.pool.engines[u].state in live)]
            rid = f"scale-out-{self._next}"
            self._next += 1
            if not urls and num_replicas <= 0:
                req = {"request_id": rid, "status": "NOOP", "message": "every named engine is already active or on its way in"}
                self.requests[rid] = req
                return dict(req)
            req = {"request_id": rid, "status": "PENDING", "engine_urls": urls, "num_replicas": int(num_replicas),
                   "timeout_secs": float(timeout_secs or self.default_timeout_s), "policy": policy or self.policy,
                   "succeeded": [], "failed": {}, "cancel": False, "message": "accepted"}
            self.requests[rid] = req
            self._busy = True
            accepted = {k: v for k, v in req.items() if k != "cancel"}
        if run_async:
            threading.Thread(target=self._execute, args=(rid,), daemon=True, name=rid).start()
            return accepted
        self._execute(rid)
        return {k: v for k, v in self.requests[rid].items() if k != "cancel"}

    def _execute(self, rid: str):
        req = self.requests[rid]
        try:
            if req["cancel"]:
                req["status"] = "CANCELLED"
                return
            req["status"] = "SYNCING"
            res = self.pool.scale_out(req["num_replicas"], req["timeout_secs"], req["policy"],
                                      ids=req["engine_urls"] or None, cancelled=lambda: req["cancel"])
            req["succeeded"], req["failed"] = [str(x) for x in res.succeeded], {str(k): v for k, v in res.failed.items()}
            if req["cancel"] and not res.succeeded:
                req["status"] = "CANCELLED"
            elif res.rolled_back or (res.failed and not res.succeeded):
                req["status"] = "FAILED"
            else:
                req["status"] = "ACTIVE" if not res.failed else "PARTIAL"
            req["message"] = f"{len(res.succeeded)} engine(s) joined, {len(res.failed)} failed"
        except Exception as e:  # noqa: BLE001 - recorded on the request
            req["status"], req["message"] = "FAILED", f"{type(e).__name__}: {e}"
        finally:
            with self._lock:
                self._busy = False

    def list(self, status: Optional[str] = None) -> list:
        return [{k: v for k, v in r.items() if k != "cancel"} for r in self.requests.values()
                if status is None or r["status"] == status.upper()]

    def cancel(self, status_filter: Optional[str] = None, dry_run: bool = False) -> list:
        hit = [r for r in self.requests.values() if r["status"] in ("PENDING", "SYNCING")
               and (status_filter is None or r["status"] == status_filter.upper())]
        if not dry_run:
            for r in hit:
                r["cancel"] = True
        return [r["request_id"] for r in hit]

    def guard(self):
        """Context for another scale operation (scale-in): refuses while a scale-out runs."""
        outer = self

        class _G:
            def __enter__(self_g):
                with outer._lock:
                    if outer._busy:
                        raise RuntimeError("CONFLICT: another scale operation is in progress")
                    outer._busy = True

            def __exit__(self_g, *a):
                with outer._lock:
                    outer._busy = False

        return _G()


class ElasticControlServer:
    def __init__(self, pool: EnginePool, host: str = "127.0.0.1", port: int = 0, autoscaler_config: Optional[str] = None,
                 metrics_fn: Optional[Callable[[], dict]] = None, on_abort: Optional[Callable[[list], None]] = None,
                 scale_out_timeout_s: float = 600.0, policy: str = "keep_partial", autoscale_interval_s: float = 0.0):
        self.pool, self.on_abort = pool, on_abort
        self.requests = ScaleRequests(pool, scale_out_timeout_s, policy)
        self.autoscaler = None
        if autoscaler_config:
            with open(autoscaler_config) as f:
                text = f.read()
            try:
                d = json.loads(text)
            except ValueError:
                import yaml

                d = yaml.safe_load(text)
            self.autoscaler = Autoscaler(pool, AutoscalerConfig.from_dict(d or {}), metrics_fn or (lambda: {}))
        srv = self

        class H(BaseHTTPRequestHandler):
            def log_message(self, *a):      # quiet
                pass

            def _reply(self, code, obj):
                body = json.dumps(obj).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def do_GET(self):
                if self.path == "/engines":
                    self._reply(200, srv.status())
                elif self.path.split("?")[0] == "/scale_out":
                    from urllib.parse import parse_qs, urlparse

                    st = parse_qs(urlparse(self.path).query).get("status", [None])[0]
                    reqs = srv.requests.list(st)
                    self._reply(200, {"requests": reqs, "total_count": len(reqs), "status_filter": st})
                elif self.path == "/health":
                    self._reply(200, {"status": "ok", "active": len(srv.pool.active())})
                elif self.path == "/metrics":          # pool gauges in Prometheus text format
                    st = [r.state.value for r in srv.pool.engines.values()]
                    rows = [("relax_rollout_engines_active", st.count("active")), ("relax_rollout_engines_draining", st.count("draining")),
                            ("relax_rollout_engines_failed", st.count("failed")),
                            ("relax_rollout_scale_requests_pending", len([r for r in srv.requests.requests.values() if r["status"] in ("PENDING", "SYNCING")]))]
                    if srv.autoscaler is not None:
                        rows.append(("relax_rollout_autoscaler_decisions_total", len(srv.autoscaler.decisions)))
                    body = "".join(f"# TYPE {n} gauge\n{n} {v}\n" for n, v in rows).encode()
                    self.send_response(200)
                    self.send_header("Content-Type", "text/plain; version=0.0.4")
                    self.send_header("Content-Length", str(len(body)))
                    self.end_headers()
                    self.wfile.write(body)
                else:
                    self._reply(404, {"error": "unknown path"})

            def do_POST(self):
                n = int(self.headers.get("Content-Length", "0") or 0)
                try:
                    req = json.loads(self.rfile.read(n) or b"{}")
                    if self.path == "/scale_out" and ("engine_urls" in req or "num_replicas" in req):
                        # request form: answers at once, the work runs in the background (GET /scale_out to follow it)
                        out = srv.requests.create(int(req.get("num_replicas", 0)), req.get("engine_urls"), req.get("timeout_secs"),
                                                  req.get("policy"))
                        self._reply(409 if out["status"] == "CONFLICT" else 200, out)
                    elif self.path == "/scale_out_cancel":
                        ids = srv.requests.cancel(req.get("status_filter"), bool(req.get("dry_run", False)))
                        self._reply(200, {"cancelled": ids, "dry_run": bool(req.get("dry_run", False))})
                    elif self.path == "/scale_out":
                        res = srv.pool.scale_out(int(req.get("num_engines", 1)), float(req.get("timeout", 600.0)),
                                                 req.get("policy", "keep_partial"))
                        self._reply(200, {"requested": res.requested, "succeeded": list(res.succeeded),
                                          "failed": {str(k): v for k, v in res.failed.items()}, "rolled_back": res.rolled_back})
                    elif self.path == "/scale_in":
                        ids = req.get("engine_ids") or [u if "://" in u else f"http://{u}" for u in req.get("engine_urls", [])] or None
                        with srv.requests.guard():
                            removed = srv.pool.scale_in(int(req.get("num_engines", req.get("num_replicas", 1))), ids=ids,
                                                        shutdown_timeout_s=float(req.get("timeout", 60.0)), on_abort=srv.on_abort)
                        self._reply(200, {"removed": list(removed)})
                    elif self.path == "/autoscale_step":
                        self._reply(200, {"action": srv.autoscaler.step() if srv.autoscaler else None})
                    else:
                        self._reply(404, {"error": "unknown path"})
                except Exception as e:  # noqa: BLE001 - a bad request must not kill the service
                    self._reply(400, {"error": f"{type(e).__name__}: {e}"})

        self.httpd = ThreadingHTTPServer((host, port), H)
        self.address = self.httpd.server_address
        threading.Thread(target=self.httpd.serve_forever, daemon=True, name="elastic-control").start()
        self._stop = threading.Event()
        if self.autoscaler is not None and autoscale_interval_s > 0:
            def loop():
                while not self._stop.wait(autoscale_interval_s):
                    try:
                        with self.requests.guard():
                            self.autoscaler.step()
                    except Exception:  # noqa: BLE001 - a failed evaluation is retried at the next tick
                        pass

            threading.Thread(target=loop, daemon=True, name="autoscaler").start()

    def status(self) -> dict:
        return {str(k): {"state": r.state.value, "weight_version": r.weight_version, "error": r.error}
                for k, r in self.pool.engines.items()}

    def close(self):
        self._stop.set()
        self.httpd.shutdown()
        self.httpd.server_close()
