"""The rollout engine behind HTTP, and a client that makes such a server look like an engine.

The reference talks to its SGLang engines over HTTP (relax/backends/sglang/sglang_engine.py: ``/generate``,
``/flush_cache``, ``/pause_generation``, ``/continue_generation``, ``/abort_request``, ``/health_generate``,
``/get_server_info``); routers, external-engine setups and elastic scale-out all build on that surface.  Here the
engine is a library object, so the server is a thin shell: one thread owns the engine and runs its scheduler loop
(``step()`` until idle), HTTP handler threads enqueue requests and wait for their results.  Requests that arrive
while a batch is running join the running batch at the next scheduler iteration (continuous batching), exactly as
in-process callers do.

``POST /generate`` body: ``{"input_ids": [..] | [[..], ..], "sampling_params": {temperature, top_p, top_k,
max_new_tokens, stop_token_ids, ignore_eos}, "routing_key": optional}`` -> per prompt ``{"output_ids", "logprobs",
"finish_reason", "weight_versions", "cached_tokens"}``.

:class:`HTTPEngine` is the client: ``generate(prompts, params)`` with the engine's own signature, against one base URL
(an engine server, or the router proxy in front of several).
"""
from __future__ import annotations

import json
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Optional, Sequence

from .engine import SamplingParams


class EngineServer:
    def __init__(self, engine, host: str = "127.0.0.1", port: int = 0, idle_sleep_s: float = 0.002, http: bool = True):
        """``http=False``: only the engine loop and the thread-safe :meth:`generate` / :meth:`command` calls (an
        in-process batching backend, e.g. under the chat endpoint that agent processes talk to)."""
        self.engine, self.idle_sleep_s = engine, idle_sleep_s
        self.httpd, self.url = None, None
        self._lock = threading.Lock()           # guards the hand-over lists; the engine itself is touched by ONE thread
        self._incoming: list = []               # (prompt, SamplingParams, group_key, ticket)
        self._commands: list = []               # (name, ticket)
        self._tickets: dict = {}                # rid -> ticket
        self._stop = threading.Event()
        self.served = 0
        self._loop = threading.Thread(target=self._run, daemon=True, name="engine-loop")
        self._loop.start()
        server = self
        if not http:
            return

        class H(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def _reply(self, code, body):
                data = json.dumps(body).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

            def do_GET(self):
                path = self.path.split("?")[0].rstrip("/")
                if path in ("/health", "/health_generate"):
                    return self._reply(200, {"status": "ok"})
                if path == "/metrics":
                    # Prometheus text format: what an external autoscaler (Prometheus + KEDA in the reference's set-up,
                    # relax/utils/autoscaler/) scrapes from every engine
                    e = server.engine
                    used = 1.0 - e.bm.num_free / max(1, e.bm.num_blocks)
                    rows = [("relax_engine_running_requests", "gauge", len(e.running)), ("relax_engine_waiting_requests", "gauge", len(e.waiting)),
                            ("relax_engine_kv_cache_usage", "gauge", round(used, 6)), ("relax_engine_weight_version", "gauge", e.weight_version),
                            ("relax_engine_requests_served_total", "counter", server.served),
                            ("relax_engine_decode_tokens_total", "counter", e.stats.get("decode_tokens", 0)),
                            ("relax_engine_prefill_tokens_total", "counter", e.stats.get("prefill_tokens", 0))]
                    text = "".join(f"# TYPE {n} {t}\n{n} {v}\n" for n, t, v in rows).encode()
                    self.send_response(200)
                    self.send_header("Content-Type", "text/plain; version=0.0.4")
                    self.send_header("Content-Length", str(len(text)))
                    self.end_headers()
                    self.wfile.write(text)
                    return None
                if path in ("/get_server_info", "/get_model_info"):
                    e = server.engine
                    return self._reply(200, {"model": e.cfg.name, "weight_version": e.weight_version, "running": len(e.running),
                                             "waiting": len(e.waiting), "kv_blocks_free": e.bm.num_free, "kv_blocks": e.bm.num_blocks,
                                             "served": server.served, "paused": bool(e.paused)})
                self._reply(404, {"error": "unknown route"})

            def do_POST(self):
                n = int(self.headers.get("Content-Length", "0") or 0)
                path = self.path.split("?")[0].rstrip("/")
                try:
                    if path == "/update_weights":
                        # body: torch.save of {name: tensor} in the engine's own layout; ?version=N
                        import io
                        from urllib.parse import parse_qs, urlparse

                        import torch

                        q = parse_qs(urlparse(self.path).query)
                        state = torch.load(io.BytesIO(self.rfile.read(n)), map_location="cpu", weights_only=True)
                        return self._reply(200, server.command("update_weights", payload=(state, int(q.get("version", ["0"])[0])),
                                                               timeout_s=600.0))
                    body = json.loads(self.rfile.read(n) or b"{}")
                    if path == "/update_weights_from_disk":
                        import torch

                        state = torch.load(body["path"], map_location="cpu", weights_only=True)
                        return self._reply(200, server.command("update_weights", payload=(state, int(body.get("weight_version", 0))),
                                                               timeout_s=600.0))
                    if path == "/generate":
                        return self._reply(200, server.generate(body))
                    if path in ("/flush_cache", "/pause_generation", "/continue_generation", "/abort_request"):
                        return self._reply(200, server.command(path[1:]))
                    self._reply(404, {"error": "unknown route"})
                except Exception as e:  # noqa: BLE001 - a bad request must not take the server down
                    self._reply(400, {"error": f"{type(e).__name__}: {e}"})

        self.httpd = ThreadingHTTPServer((host, port), H)
        self.url = f"http://{host}:{self.httpd.server_address[1]}"
        threading.Thread(target=self.httpd.serve_forever, daemon=True, name="engine-http").start()

    # ------------------------------------------------------------------ handler side
    def generate(self, body: dict, timeout_s: float = 3600.0):
        ids = body["input_ids"]
        many = bool(ids) and isinstance(ids[0], (list, tuple))
        prompts = ids if many else [ids]
        sp = body.get("sampling_params") or {}
        params = SamplingParams(temperature=float(sp.get("temperature", 1.0)), top_p=float(sp.get("top_p", 1.0)),
                                top_k=int(sp.get("top_k", -1)), max_new_tokens=int(sp.get("max_new_tokens", 128)),
                                stop_token_ids=tuple(sp.get("stop_token_ids") or ()), ignore_eos=bool(sp.get("ignore_eos", False)))
        key = body.get("routing_key")
        tickets = []
        with self._lock:
            for p in prompts:
                t = {"event": threading.Event(), "result": None}
                self._incoming.append(([int(x) for x in p], params, key, t))
                tickets.append(t)
        out = []
        for t in tickets:
            if not t["event"].wait(timeout_s):
                raise TimeoutError("generation did not finish in time")
            out.append(t["result"])
        return out if many else out[0]

    def command(self, name: str, timeout_s: float = 60.0, payload=None):
        t = {"event": threading.Event(), "result": None, "payload": payload}
        with self._lock:
            self._commands.append((name, t))
        if not t["event"].wait(timeout_s):
            raise TimeoutError(f"{name} was not executed in time")
        return t["result"]

    # ------------------------------------------------------------------ the one thread that owns the engine
    def _finish(self, r):
        t = self._tickets.pop(r.rid, None)
        if t is None:
            return
        t["result"] = {"output_ids": list(r.output), "logprobs": [float(x) for x in r.logprobs], "finish_reason": r.finish_reason,
                       "weight_versions": sorted(set(r.weight_versions)), "cached_tokens": int(r.cached_tokens)}
        self.served += 1
        t["event"].set()

    def _run(self):
        eng = self.engine
        dev = getattr(eng, "device", None)
        if dev is not None and getattr(dev, "type", "cpu") == "cuda":
            import torch

            torch.cuda.set_device(dev)        # the current device is per thread
        while not self._stop.is_set():
            with self._lock:
                incoming, self._incoming = self._incoming, []
                commands, self._commands = self._commands, []
            for name, t in commands:
                if name == "flush_cache":
                    ok = not eng.running
                    if ok:
                        eng.flush_cache()
                    t["result"] = {"status": "ok" if ok else "busy"}
                elif name == "pause_generation":
                    eng.pause_generation()
                    t["result"] = {"status": "ok"}
                elif name == "continue_generation":
                    eng.continue_generation()
                    t["result"] = {"status": "ok"}
                elif name == "update_weights":
                    # between scheduler iterations: running requests continue with the new weights and record both
                    # versions, exactly as with an in-process sync
                    state, version = t["payload"]
                    try:
                        missing = [k for k in eng.weights.p if k not in state]
                        extra = [k for k in state if k not in eng.weights.p]
                        if missing or extra:
                            raise KeyError(f"weight names differ: missing {missing[:3]}, unexpected {extra[:3]}")
                        import torch

                        with torch.no_grad():
                            for k, v in state.items():
                                dst = eng.weights.p[k]
                                if tuple(dst.shape) != tuple(v.shape):
                                    raise ValueError(f"{k}: shape {tuple(v.shape)} does not fit {tuple(dst.shape)}")
                                dst.copy_(v.to(dst.dtype))
                        if not eng.running:
                            eng.flush_cache()
                        eng.update_weight_version(version)
                        t["result"] = {"status": "ok", "weight_version": version, "tensors": len(state)}
                    except Exception as e:  # noqa: BLE001 - reported to the caller, the server keeps its old weights
                        t["result"] = {"status": "error", "error": f"{type(e).__name__}: {e}"}
                elif name == "abort_request":
                    done = eng.abort_all()
                    for r in done:
                        self._finish(r)
                    t["result"] = {"status": "ok", "aborted": len(done)}
                t["event"].set()
            for prompt, params, key, t in incoming:
                rid = eng.add_request(prompt, params, key)
                self._tickets[rid] = t
            if eng.has_work and not eng.paused:
                try:
                    for r in eng.step():
                        self._finish(r)
                except Exception as e:  # noqa: BLE001 - fail the requests in flight, keep serving
                    for r in eng.abort_all():
                        r.finish_reason = f"error: {type(e).__name__}: {e}"
                        self._finish(r)
            else:
                time.sleep(self.idle_sleep_s)

    def close(self):
        self._stop.set()
        if self.httpd is not None:
            self.httpd.shutdown()
            self.httpd.server_close()
        self._loop.join(timeout=5)

    def generate_fn(self, sampling):
        """The engine loop as a ``generate(prompts, max_new_tokens, group_keys)`` callable (the signature the agentic
        code uses); calls from several threads join one running batch."""
        sp = {"temperature": sampling.temperature, "top_p": sampling.top_p, "top_k": sampling.top_k,
              "stop_token_ids": list(sampling.stop_token_ids), "ignore_eos": sampling.ignore_eos}

        def gen(prompts, max_new, keys):
            outs = []
            # one request list per routing key keeps the prefix-sharing groups of the engine intact
            body = {"input_ids": [list(p) for p in prompts], "sampling_params": dict(sp, max_new_tokens=int(max_new)),
                    "routing_key": keys[0] if keys and len(set(keys)) == 1 else None}
            for d in self.generate(body):
                outs.append((d["output_ids"], d["logprobs"], d["finish_reason"], d["weight_versions"]))
            return outs

        return gen


class _Result:
    """What :meth:`RolloutEngine.generate` returns per prompt, rebuilt from the server's answer."""

    def __init__(self, prompt, d):
        self.prompt, self.output, self.logprobs = list(prompt), list(d["output_ids"]), list(d["logprobs"])
        self.finish_reason, self.weight_versions = d.get("finish_reason"), list(d.get("weight_versions") or [])
        self.cached_tokens, self.routed_experts = int(d.get("cached_tokens", 0)), []


class HTTPEngine:
    """An engine server (or the router in front of several) used through the engine's ``generate`` call."""

    def __init__(self, url: str, timeout_s: float = 3600.0):
        self.url, self.timeout_s = url.rstrip("/"), timeout_s

    def _post(self, path: str, obj: dict):
        import urllib.request

        req = urllib.request.Request(self.url + path, data=json.dumps(obj).encode(), headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
            return json.loads(r.read().decode())

    def generate(self, prompts: Sequence[Sequence[int]], params, group_keys: Optional[Sequence] = None, images=None):
        if images is not None and any(images):
            raise NotImplementedError("image prompts do not travel over the HTTP surface")
        sp = params if isinstance(params, SamplingParams) else params[0]
        body = {"input_ids": [list(map(int, p)) for p in prompts],
                "sampling_params": {"temperature": sp.temperature, "top_p": sp.top_p, "top_k": sp.top_k, "max_new_tokens": sp.max_new_tokens,
                                    "stop_token_ids": list(sp.stop_token_ids), "ignore_eos": sp.ignore_eos}}
        return [_Result(p, d) for p, d in zip(prompts, self._post("/generate", body))]

    def flush_cache(self):
        return self._post("/flush_cache", {})

    def info(self) -> dict:
        import urllib.request

        with urllib.request.urlopen(self.url + "/get_server_info", timeout=30.0) as r:
            return json.loads(r.read().decode())

    def update_weights(self, state: dict, version: int) -> dict:
        """Ship ``{name: tensor}`` (the engine's layout) in the request body."""
        import io
        import urllib.request

        import torch

        buf = io.BytesIO()
        torch.save({k: v.detach().to("cpu") for k, v in state.items()}, buf)
        req = urllib.request.Request(f"{self.url}/update_weights?version={int(version)}", data=buf.getvalue(),
                                     headers={"Content-Type": "application/octet-stream"})
        with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
            out = json.loads(r.read().decode())
        if out.get("status") != "ok":
            raise RuntimeError(f"{self.url} refused the weights: {out.get('error', out)}")
        return out

    def health(self) -> bool:
        import urllib.request

        try:
            with urllib.request.urlopen(self.url + "/health", timeout=5.0) as r:
                return r.status == 200
        except Exception:  # noqa: BLE001
            return False
