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


class ElasticControlServer:
    def __init__(self, pool: EnginePool, host: str = "127.0.0.1", port: int = 0, autoscaler_config: Optional[str] = None,
                 metrics_fn: Optional[Callable[[], dict]] = None, on_abort: Optional[Callable[[list], None]] = None):
        self.pool, self.on_abort = pool, on_abort
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
                elif self.path == "/health":
                    self._reply(200, {"status": "ok", "active": len(srv.pool.active())})
                else:
                    self._reply(404, {"error": "unknown path"})

            def do_POST(self):
                n = int(self.headers.get("Content-Length", "0") or 0)
                try:
                    req = json.loads(self.rfile.read(n) or b"{}")
                    if self.path == "/scale_out":
                        res = srv.pool.scale_out(int(req.get("num_engines", 1)), float(req.get("timeout", 600.0)),
                                                 req.get("policy", "keep_partial"))
                        self._reply(200, {"requested": res.requested, "succeeded": list(res.succeeded),
                                          "failed": {str(k): v for k, v in res.failed.items()}, "rolled_back": res.rolled_back})
                    elif self.path == "/scale_in":
                        removed = srv.pool.scale_in(int(req.get("num_engines", 1)), ids=req.get("engine_ids"),
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

    def status(self) -> dict:
        return {str(k): {"state": r.state.value, "weight_version": r.weight_version, "error": r.error}
                for k, r in self.pool.engines.items()}

    def close(self):
        self.httpd.shutdown()
        self.httpd.server_close()
