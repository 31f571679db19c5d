"""Request router in front of the rollout engines: least-loaded choice, sticky routing by key (all
samples of a prompt group, or all turns of an agent session, land on the engine that holds their
prefix), periodic health checks with quarantine, and worker add/remove for elastic scale-out/in.

Behaviour follows the reference router (relax/engine/router/router.py:152-316): a worker's load is
its number of requests in flight; a sticky key keeps its worker while that worker is healthy and is
forgotten after ``sticky_idle_s`` without use; a worker that fails ``max_failures`` consecutive
probes is quarantined and its sticky keys are released.  Workers are opaque handles (an in-process
engine, a URL); the transport is the caller's.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional


@dataclass
class WorkerState:
    handle: object
    in_flight: int = 0
    healthy: bool = True
    consecutive_failures: int = 0
    served: int = 0
    draining: bool = False     # scale-in: finish what it has, accept nothing new


class NoHealthyWorker(RuntimeError):
    pass


class Router:
    def __init__(self, max_failures: int = 3, sticky_idle_s: float = 600.0, clock: Callable[[], float] = time.monotonic):
        self._workers: Dict[Hashable, WorkerState] = {}
        self._sticky: Dict[Hashable, tuple] = {}    # key -> (worker id, last use)
        self._lock = threading.Lock()
        self.max_failures, self.sticky_idle_s, self._clock = max_failures, sticky_idle_s, clock
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    # ------------------------------------------------------------------ membership
    def add_worker(self, wid: Hashable, handle: object = None):
        with self._lock:
            self._workers[wid] = WorkerState(handle if handle is not None else wid)

    def remove_worker(self, wid: Hashable):
        with self._lock:
            self._workers.pop(wid, None)
            self._sticky = {k: v for k, v in self._sticky.items() if v[0] != wid}

    def drain_worker(self, wid: Hashable):
        """Stop sending new requests to ``wid`` (scale-in); :meth:`is_idle` tells when it can go."""
        with self._lock:
            if wid in self._workers:
                self._workers[wid].draining = True
            self._sticky = {k: v for k, v in self._sticky.items() if v[0] != wid}

    def is_idle(self, wid: Hashable) -> bool:
        with self._lock:
            w = self._workers.get(wid)
            return w is None or w.in_flight == 0

    def workers(self) -> Dict[Hashable, dict]:
        with self._lock:
            return {k: {"in_flight": w.in_flight, "healthy": w.healthy, "served": w.served, "draining": w.draining}
                    for k, w in self._workers.items()}

    # ------------------------------------------------------------------ routing
    def _eligible(self) -> List[Hashable]:
        return [k for k, w in self._workers.items() if w.healthy and not w.draining]

    def acquire(self, routing_key: Optional[Hashable] = None) -> Hashable:
        """Pick the worker of the next request and count it as in flight; pair with :meth:`release`."""
        with self._lock:
            now = self._clock()
            self._sticky = {k: v for k, v in self._sticky.items() if now - v[1] <= self.sticky_idle_s}
            ok = self._eligible()
            if not ok:
                raise NoHealthyWorker("no healthy rollout engine to route to")
            wid = None
            if routing_key is not None and routing_key in self._sticky and self._sticky[routing_key][0] in ok:
                wid = self._sticky[routing_key][0]
            if wid is None:
                wid = min(ok, key=lambda k: (self._workers[k].in_flight, self._workers[k].served))
            if routing_key is not None:
                self._sticky[routing_key] = (wid, now)
            w = self._workers[wid]
            w.in_flight += 1
            w.served += 1
            return wid

    def release(self, wid: Hashable, failed: bool = False):
        with self._lock:
            w = self._workers.get(wid)
            if w is None:
                return
            w.in_flight = max(0, w.in_flight - 1)
            if failed:
                self._note_failure(wid, w)

    def quarantine(self, wid: Hashable):
        """Take ``wid`` out of rotation now (a request to it failed outright); health probes readmit it."""
        with self._lock:
            w = self._workers.get(wid)
            if w is not None and w.healthy:
                w.healthy = False
                w.consecutive_failures = max(w.consecutive_failures, self.max_failures)
                self._sticky = {k: v for k, v in self._sticky.items() if v[0] != wid}

    def readmit(self, wid: Hashable):
        """Put ``wid`` back into rotation (its owner has checked it and brought it up to date)."""
        with self._lock:
            w = self._workers.get(wid)
            if w is not None:
                w.healthy, w.consecutive_failures = True, 0

    def handle(self, wid: Hashable):
        return self._workers[wid].handle

    # ------------------------------------------------------------------ health
    def _note_failure(self, wid, w: WorkerState):
        w.consecutive_failures += 1
        if w.consecutive_failures >= self.max_failures and w.healthy:
            w.healthy = False
            self._sticky = {k: v for k, v in self._sticky.items() if v[0] != wid}

    def check_health(self, probe: Callable[[object], bool]):
        """One round of probes (``probe(handle) -> bool``); a quarantined worker that answers again is readmitted."""
        with self._lock:
            items = list(self._workers.items())
        for wid, w in items:
            try:
                ok = bool(probe(w.handle))
            except Exception:  # noqa: BLE001
                ok = False
            with self._lock:
                if wid not in self._workers:
                    continue
                if ok:
                    w.consecutive_failures, w.healthy = 0, True
                else:
                    self._note_failure(wid, w)

    def start_health_loop(self, probe: Callable[[object], bool], interval_s: float = 10.0):
        def loop():
            while not self._stop.wait(interval_s):
                self.check_health(probe)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)


# ----------------------------------------------------------------------------- HTTP front
def serve_router(router: Optional[Router] = None, host: str = "127.0.0.1", port: int = 0, timeout_s: float = 600.0,
                 health_path: str = "/health", health_interval_s: float = 10.0, retries: int = 2):
    """The router as an HTTP proxy in front of engine servers (relax/engine/router/router.py: ``/add_worker``,
    ``/remove_worker``, ``/list_workers``, and every other POST forwarded to a worker).  Workers are base URLs.
    A forwarded request goes to the least-loaded healthy worker - or to the worker that already holds the request's
    ``routing_key`` / ``session_id`` / ``user`` field - and is retried on another worker when the first fails;
    ``GET <worker><health_path>`` probes run in the background and quarantine a worker after ``max_failures`` misses.
    Returns ``(server, thread, router)``."""
    import json
    import urllib.error
    import urllib.parse
    import urllib.request
    from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

    router = router or Router()

    def probe(url) -> bool:
        try:
            with urllib.request.urlopen(str(url).rstrip("/") + health_path, timeout=5.0) as r:
                return 200 <= r.status < 300
        except Exception:  # noqa: BLE001
            return False

    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def _send(self, code, body: bytes, ctype="application/json"):
            self.send_response(code)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def _json(self, code, obj):
            self._send(code, json.dumps(obj).encode())

        def _url_arg(self, body: bytes) -> Optional[str]:
            q = urllib.parse.parse_qs(urllib.parse.urlparse(self.path).query)
            if "url" in q:
                return q["url"][0]
            try:
                return json.loads(body.decode() or "{}").get("url")
            except ValueError:
                return None

        def do_GET(self):
            path = urllib.parse.urlparse(self.path).path.rstrip("/")
            if path == "/list_workers":
                return self._json(200, {"urls": [str(w) for w in router.workers()], "workers": {str(k): v for k, v in router.workers().items()}})
            if path == "/health":
                return self._json(200, {"status": "ok", "workers": len(router.workers())})
            self._json(404, {"error": "not found"})

        def do_POST(self):
            body = self.rfile.read(int(self.headers.get("Content-Length", "0") or 0))
            path = urllib.parse.urlparse(self.path).path.rstrip("/")
            if path in ("/add_worker", "/remove_worker", "/drain_worker"):
                url = self._url_arg(body)
                if not url:
                    return self._json(400, {"error": "url missing"})
                {"/add_worker": router.add_worker, "/remove_worker": router.remove_worker, "/drain_worker": router.drain_worker}[path](url)
                return self._json(200, {"status": "ok", "urls": [str(w) for w in router.workers()]})
            key = None
            try:
                d = json.loads(body.decode() or "{}")
                key = d.get("routing_key") or d.get("session_id") or d.get("user")
            except ValueError:
                pass
            last = None
            for _ in range(retries + 1):
                try:
                    wid = router.acquire(key)
                except NoHealthyWorker as e:
                    return self._json(503, {"error": str(e)})
                failed = True
                try:
                    req = urllib.request.Request(str(router.handle(wid)).rstrip("/") + self.path, data=body,
                                                 headers={"Content-Type": self.headers.get("Content-Type", "application/json")})
                    with urllib.request.urlopen(req, timeout=timeout_s) as r:
                        out, code, ctype = r.read(), r.status, r.headers.get("Content-Type", "application/json")
                    failed = False
                    return self._send(code, out, ctype)
                except urllib.error.HTTPError as e:      # the worker answered: pass its verdict on, it is not down
                    failed = e.code >= 500
                    last = e
                    if not failed:
                        return self._send(e.code, e.read(), e.headers.get("Content-Type", "application/json"))
                except Exception as e:  # noqa: BLE001 - connection refused / reset / timeout: try another worker
                    last = e
                finally:
                    router.release(wid, failed=failed)
            self._json(502, {"error": f"no worker could serve the request: {last!r}"})

    srv = ThreadingHTTPServer((host, port), H)
    t = threading.Thread(target=srv.serve_forever, daemon=True, name="router-http")
    t.start()
    if health_interval_s and health_interval_s > 0:
        router.start_health_loop(probe, health_interval_s)
    return srv, t, router
