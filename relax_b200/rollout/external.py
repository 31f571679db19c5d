"""Engines that somebody else started: ``--rollout-external --rollout-external-engine-addrs host:port ...``.

The training job neither launches nor stops these servers (``python -m relax_b200.entrypoints.serve engine``); it
checks that they serve the model it trains, generates through them and keeps their weights current
(relax/backends/sglang/sglang_engine.py:494-499 ``_init_external`` and :844 ``shutdown`` - no process of its own;
relax/distributed/ray/rollout.py:4073-4083 - engine rank ``r`` uses address ``r`` of the list).

:class:`ExternalEngine` has the surface the colocated loop and :class:`~relax_b200.weight_sync.sync.WeightSync` use of
an in-process engine.  Weight updates go through a staging copy: the sync writes the trainer's weights, converted to
the engines' layout, into ``self.weights`` on the trainer's device exactly as it would into a local engine;
``update_weight_version`` then ships that buffer to every server (one HTTP request per server, in parallel) and the
servers apply it between two scheduler iterations.  The staging copy costs one set of weights in device memory; it is
what lets every trainer layout (TP, PP, EP) reuse the block-copy plans unchanged.
"""
from __future__ import annotations

import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Optional, Sequence

from .http_server import HTTPEngine


def _guard(fn, arg):
    try:
        fn(arg)
        return None
    except Exception as e:  # noqa: BLE001 - reported per server by the caller
        return e


class ExternalEngine:
    def __init__(self, cfg, addrs: Sequence[str], device, dtype, max_model_len: Optional[int] = None, timeout_s: float = 3600.0,
                 check_fields: Sequence[str] = ("model",)):
        from .weights import RolloutWeights

        if not addrs:
            raise ValueError("--rollout-external needs --rollout-external-engine-addrs")
        if cfg.vision is not None:
            raise NotImplementedError("image prompts do not travel over the HTTP surface: external engines serve text models")
        self.cfg, self.device, self.dtype, self.max_model_len = cfg, device, dtype, max_model_len
        from .router import Router

        self.timeout_s, self.check_fields = timeout_s, tuple(check_fields)
        self.max_retries = 3                     # rounds of re-routing the prompt groups of servers that failed
        self.router = Router()                                           # membership, load, draining, health of the servers
        clients = [self.connect(a) for a in addrs]
        self.weights = RolloutWeights(cfg, 1, 0, device, dtype)          # staging, in the servers' layout (TP 1)
        self.weight_version = 0
        self.running: list = []
        self.paused = False
        self.bm = None                                                   # no local KV cache
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "cached_tokens": 0, "steps": 0}
        self._pool = ThreadPoolExecutor(max_workers=16, thread_name_prefix="ext-engine")
        self._lock = threading.Lock()
        for c in clients:
            self.router.add_worker(c.url, c)

    # ------------------------------------------------------------------ membership
    def connect(self, addr: str) -> HTTPEngine:
        """A client for ``addr`` after checking that the server answers and serves what this job trains."""
        c = HTTPEngine(addr if "://" in addr else f"http://{addr}", self.timeout_s)
        info = c.info()
        for f in self.check_fields:
            want = {"model": self.cfg.name}.get(f)
            if want is not None and info.get(f) != want:
                raise ValueError(f"{c.url} serves {f}={info.get(f)!r}, this job trains {want!r}")
        return c

    @property
    def clients(self) -> list:
        """The servers that currently take requests and weight updates (draining ones included until removed)."""
        return [self.router.handle(k) for k in self.router.workers()]

    def ship_current_weights(self, client: HTTPEngine) -> int:
        """Bring one server to the staging buffer's version (a server that joins while training runs)."""
        v = self.weight_version
        client.update_weights({k: t.detach().to("cpu") for k, t in self.weights.p.items()}, v)
        return v

    def server_metrics(self) -> dict:
        """Gauges for autoscaling rules, from the servers' own status pages."""
        infos = []
        for c in self.clients:
            try:
                infos.append(c.info())
            except Exception:  # noqa: BLE001 - a dead server is the health loop's business
                pass
        n = max(1, len(infos))
        used = sum(1.0 - i.get("kv_blocks_free", 0) / max(1, i.get("kv_blocks", 1)) for i in infos)
        return {"queue_depth_per_engine": sum(i.get("waiting", 0) for i in infos) / n,
                "running_per_engine": sum(i.get("running", 0) for i in infos) / n,
                "kv_cache_utilization": used / n, "num_engines": float(len(infos))}

    def readmit_recovered(self) -> list:
        """Servers that were taken out of rotation and answer again get the CURRENT weights and only then requests."""
        back = []
        for wid, w in self.router.workers().items():
            if w["healthy"]:
                continue
            c = self.router.handle(wid)
            try:
                if c.health():
                    self.ship_current_weights(c)
                    self.router.readmit(wid)
                    back.append(wid)
            except Exception:  # noqa: BLE001 - still down
                pass
        return back

    # ------------------------------------------------------------------ what WeightSync calls
    def _all(self, fn):
        """``fn`` on every server in rotation; one that fails is taken out (it is brought up to date when it returns)."""
        live = [(wid, self.router.handle(wid)) for wid, w in self.router.workers().items() if w["healthy"]]
        if not live:
            raise RuntimeError("no external engine is reachable")
        res = list(self._pool.map(lambda it: _guard(lambda c: fn(c), it[1]), live))
        bad = [wid for (wid, _), r in zip(live, res) if r is not None]
        for wid in bad:
            self.router.quarantine(wid)
        if len(bad) == len(live):
            raise RuntimeError(f"every external engine failed: {[r for r in res if r is not None][0]}")
        return res

    def pause_generation(self):
        self.paused = True
        self._all(lambda c: c._post("/pause_generation", {}))

    def continue_generation(self):
        self._all(lambda c: c._post("/continue_generation", {}))
        self.paused = False

    def flush_cache(self):
        self._all(lambda c: c.flush_cache())

    def update_weight_version(self, v: int):
        """The staging buffer holds version ``v``: push it to every server."""
        state = {k: t.detach().to("cpu") for k, t in self.weights.p.items()}      # one device read, shared by the requests
        self._all(lambda c: c.update_weights(state, int(v)))
        self.weight_version = int(v)

    # ------------------------------------------------------------------ what the rollout loop calls
    def generate(self, prompts, params, group_keys=None, images=None):
        """Prompt groups are kept together (prefix sharing on the server) and spread over the servers by load; the groups
        of a server that fails are generated again on the others.  Results come back in the order of ``prompts``."""
        if images is not None and any(images):
            raise NotImplementedError("image prompts do not travel over the HTTP surface")
        if any(not w["healthy"] for w in self.router.workers().values()):
            self.readmit_recovered()
        n = len(prompts)
        keys = list(group_keys) if group_keys is not None else list(range(n))
        groups: dict = {}
        for i in range(n):
            groups.setdefault(keys[i], []).append(i)
        out = [None] * n

        def run(item):
            wid, idx = item
            sp = params if not isinstance(params, (list, tuple)) else params[idx[0]]
            for i, r in zip(idx, self.router.handle(wid).generate([prompts[i] for i in idx], sp)):
                out[i] = r

        todo, err, attempt = dict(groups), None, 0
        while todo:
            # the router picks a server per prompt group: least loaded among the healthy ones that are not draining
            shares: dict = {}
            taken = []
            for key, idx in todo.items():
                wid = self.router.acquire(key)          # raises NoHealthyWorker when nothing is left to try
                taken.append(wid)
                shares.setdefault(wid, []).extend(idx)
            failed = set()
            try:
                for (wid, _), res in zip(shares.items(), self._pool.map(lambda it: _guard(run, it), list(shares.items()))):
                    if res is not None:
                        failed.add(wid)
                        err = res
            finally:
                for wid in taken:
                    self.router.release(wid, failed=wid in failed)
            # prompt groups of a server that failed go to the others; a server that keeps failing is quarantined by the
            # router (and comes back when it answers health probes again)
            todo = {key: idx for key, idx in todo.items() if any(out[i] is None for i in idx)}
            if todo:
                attempt += 1
                self.stats["failovers"] = self.stats.get("failovers", 0) + len(todo)
                for wid in failed:
                    self.router.quarantine(wid)
                if attempt > self.max_retries:
                    raise RuntimeError(f"external engine(s) {sorted(failed)} failed: {err}")
        with self._lock:
            self.stats["decode_tokens"] += sum(len(r.output) for r in out)
            self.stats["prefill_tokens"] += sum(len(p) for p in prompts)
            self.stats["cached_tokens"] += sum(r.cached_tokens for r in out)
        return out

    def abort_all(self) -> list:
        self._all(lambda c: c._post("/abort_request", {}))
        return []

    @property
    def has_work(self) -> bool:
        return False

    def attach_vision(self, tower):
        raise NotImplementedError("external engines serve text models")

    def release_memory_occupation(self, tags=()):          # the servers own their memory
        pass

    def resume_memory_occupation(self, tags=()):
        pass

    def close(self):
        self._pool.shutdown(wait=False)                    # the servers keep running: they are not ours


def external_pool(engine: ExternalEngine, standby: Sequence[str] = (), precheck: bool = True):
    """An :class:`~relax_b200.rollout.elastic.EnginePool` over the servers of ``engine``: scale-out connects further
    servers (named by URL, or the next of ``standby``), checks them, ships the CURRENT weights and only then lets
    the router send them requests; scale-in drains a server and forgets it (it keeps running: it is not ours).
    relax/distributed/ray/rollout.py create_scale_out_request / execute_scale_out (external mode)."""
    from .elastic import EnginePool
    from .engine import SamplingParams

    spare = [a if "://" in a else f"http://{a}" for a in standby]

    def factory(eid):
        return engine.connect(eid)

    def next_standby():
        with engine._lock:
            if not spare:
                raise RuntimeError("no standby engine address left to scale out to")
            return spare.pop(0)

    def check(seed, new) -> bool:
        if not precheck:
            return True
        try:
            return new.health() and len(new.generate([[1, 2]], SamplingParams(temperature=0.0, max_new_tokens=1))[0].output) == 1
        except Exception:  # noqa: BLE001
            return False

    def release_addr(client):
        with engine._lock:
            if client is not None and client.url not in spare:
                spare.append(client.url)             # may be scaled out to again later

    pool = EnginePool(engine.router, factory, lambda seed, new: engine.ship_current_weights(new), precheck=check,
                      shutdown=release_addr, abort=lambda c: c._post("/abort_request", {}) and [])
    for url in list(engine.router.workers()):
        from .elastic import EngineRecord, EngineState

        pool.engines[url] = EngineRecord(engine.router.handle(url), EngineState.ACTIVE, engine.weight_version, pool.clock())
    pool.next_id = next_standby
    pool.external = engine
    return pool
