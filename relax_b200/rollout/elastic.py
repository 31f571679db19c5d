"""Elastic rollout: a pool of engines that grows and shrinks while training runs, and the
rule-based autoscaler that drives it.

Scale-out (relax/distributed/ray/rollout.py:1453-3500): create the new engines, run a
communication precheck against the seed engine, copy the CURRENT weights from a healthy seed engine
(engine-to-engine, the trainer is not involved), then admit them to the router.  A request either
succeeds for all engines or, by policy, keeps the ones that made it (``keep_partial``) or rolls all
of them back (``rollback_all``).  Scale-in (:3500-3920): stop routing to the chosen engines, let
their requests finish up to a timeout, abort what is left (partial samples go back to the buffer
through ``on_abort``) and shut them down.  The autoscaler (relax/utils/autoscaler/) evaluates
threshold rules with a hold time and cooldowns over metrics the caller supplies.
"""
from __future__ import annotations

import enum
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence

from .router import Router


class EngineState(str, enum.Enum):
    PENDING = "pending"
    SYNCING = "syncing"
    ACTIVE = "active"
    DRAINING = "draining"
    REMOVED = "removed"
    FAILED = "failed"


@dataclass
class EngineRecord:
    engine: object
    state: EngineState = EngineState.PENDING
    weight_version: int = -1
    created_at: float = 0.0
    error: Optional[str] = None


@dataclass
class ScaleResult:
    requested: int
    succeeded: List[Hashable] = field(default_factory=list)
    failed: Dict[Hashable, str] = field(default_factory=dict)
    rolled_back: bool = False


class EnginePool:
    def __init__(self, router: Router, factory: Callable[[Hashable], object], sync_weights: Callable[[object, object], int],
                 precheck: Optional[Callable[[object, object], bool]] = None, shutdown: Optional[Callable[[object], None]] = None,
                 abort: Optional[Callable[[object], list]] = None, clock: Callable[[], float] = time.monotonic,
                 sleep: Callable[[float], None] = time.sleep):
        self.router, self.factory, self.sync_weights = router, factory, sync_weights
        self.precheck, self.shutdown, self.abort = precheck, shutdown, abort
        self.clock, self.sleep = clock, sleep
        self.engines: Dict[Hashable, EngineRecord] = {}
        self.next_id: Optional[Callable[[], Hashable]] = None      # names the engines of a count-based scale-out
        self._next = 0
        self._lock = threading.Lock()

    # ------------------------------------------------------------------ bookkeeping
    def add_existing(self, eid: Hashable, engine, weight_version: int = 0):
        self.engines[eid] = EngineRecord(engine, EngineState.ACTIVE, weight_version, self.clock())
        self.router.add_worker(eid, engine)

    def active(self) -> List[Hashable]:
        return [k for k, r in self.engines.items() if r.state == EngineState.ACTIVE]

    def _seed(self) -> Optional[Hashable]:
        act = self.active()
        return max(act, key=lambda k: self.engines[k].weight_version) if act else None

    def set_weight_version(self, version: int):
        for r in self.engines.values():
            if r.state == EngineState.ACTIVE:
                r.weight_version = version

    # ------------------------------------------------------------------ scale out
    def scale_out(self, n: int, timeout_s: float = 600.0, partial_success_policy: str = "keep_partial",
                  ids: Optional[Sequence[Hashable]] = None, cancelled: Optional[Callable[[], bool]] = None) -> ScaleResult:
        """``ids``: explicit engine ids (addresses of engines that already run) instead of ``n`` new ones; ids that
        are active or on their way in are skipped, so that a repeated request changes nothing.  ``cancelled()`` is
        polled between engines; engines not yet started when it turns true are not started."""
        if partial_success_policy not in ("keep_partial", "rollback_all"):
            raise ValueError("partial_success_policy is keep_partial or rollback_all")
        if ids is not None:
            live = (EngineState.ACTIVE, EngineState.PENDING, EngineState.SYNCING)
            ids = [i for i in dict.fromkeys(ids) if not (i in self.engines and self.engines[i].state in live)]
            n = len(ids)
        res = ScaleResult(requested=n)
        if n == 0:
            return res
        seed_id = self._seed()
        if seed_id is None:
            raise RuntimeError("scale-out needs at least one active engine to copy the weights from")
        seed = self.engines[seed_id]
        deadline = self.clock() + timeout_s
        new_ids = []
        for j in range(n):
            if cancelled is not None and cancelled():
                break
            with self._lock:
                if ids is not None:
                    eid = ids[j]
                elif self.next_id is not None:
                    try:
                        eid = self.next_id()           # e.g. the next address of a standby list
                    except Exception as e:  # noqa: BLE001 - nothing left to scale out to
                        res.failed[f"scaled-{self._next}"] = f"{type(e).__name__}: {e}"
                        self._next += 1
                        break
                else:
                    eid = f"scaled-{self._next}"
                    self._next += 1
            rec = EngineRecord(None, EngineState.PENDING, -1, self.clock())
            self.engines[eid] = rec
            new_ids.append(eid)
            try:
                if self.clock() > deadline:
                    raise TimeoutError("scale-out timed out before this engine was created")
                rec.engine = self.factory(eid)
                if self.precheck is not None and not self.precheck(seed.engine, rec.engine):
                    raise RuntimeError("communication precheck with the seed engine failed")
                rec.state = EngineState.SYNCING
                rec.weight_version = self.sync_weights(seed.engine, rec.engine)
                if self.clock() > deadline:
                    raise TimeoutError("scale-out timed out during the weight copy")
                res.succeeded.append(eid)
            except Exception as e:  # noqa: BLE001
                rec.state, rec.error = EngineState.FAILED, f"{type(e).__name__}: {e}"
                res.failed[eid] = rec.error
        if res.failed and partial_success_policy == "rollback_all":
            for eid in res.succeeded:
                self._dispose(eid)
            res.succeeded, res.rolled_back = [], True
        for eid in res.succeeded:
            # an engine whose copy raced with a weight update is behind the seed: refresh before admitting it
            if self.engines[eid].weight_version < seed.weight_version:
                self.engines[eid].weight_version = self.sync_weights(seed.engine, self.engines[eid].engine)
            self.engines[eid].state = EngineState.ACTIVE
            self.router.add_worker(eid, self.engines[eid].engine)
        for eid in res.failed:
            self._dispose(eid, keep_record=True)
        return res

    def _dispose(self, eid, keep_record: bool = False):
        rec = self.engines.get(eid)
        if rec is None:
            return
        if rec.engine is not None and self.shutdown is not None:
            try:
                self.shutdown(rec.engine)
            except Exception:  # noqa: BLE001
                pass
        self.router.remove_worker(eid)
        if keep_record:
            rec.engine = None
        else:
            rec.state = EngineState.REMOVED
            rec.engine = None

    # ------------------------------------------------------------------ scale in
    def scale_in(self, n: int = 1, ids: Optional[Sequence[Hashable]] = None, shutdown_timeout_s: float = 60.0,
                 on_abort: Optional[Callable[[list], None]] = None, min_engines: int = 1) -> List[Hashable]:
        act = self.active()
        if ids is None:
            loads = self.router.workers()
            # newest and least loaded first; never below ``min_engines``
            cands = sorted(act, key=lambda k: (loads.get(k, {}).get("in_flight", 0), -self.engines[k].created_at))
            ids = cands[:max(0, min(n, len(act) - min_engines))]
        removed = []
        for eid in ids:
            rec = self.engines.get(eid)
            if rec is None or rec.state != EngineState.ACTIVE:
                continue
            rec.state = EngineState.DRAINING
            self.router.drain_worker(eid)
        deadline = self.clock() + shutdown_timeout_s
        pending = [e for e in ids if e in self.engines and self.engines[e].state == EngineState.DRAINING]
        while pending and self.clock() < deadline:
            pending = [e for e in pending if not self.router.is_idle(e)]
            if pending:
                self.sleep(0.05)
        for eid in ids:
            rec = self.engines.get(eid)
            if rec is None or rec.state != EngineState.DRAINING:
                continue
            if not self.router.is_idle(eid) and self.abort is not None:
                partial = self.abort(rec.engine)
                if partial and on_abort is not None:
                    on_abort(partial)
            self._dispose(eid)
            removed.append(eid)
        return removed

    # ------------------------------------------------------------------ eviction of dead engines
    def evict_unhealthy(self) -> List[Hashable]:
        w = self.router.workers()
        dead = [k for k in self.active() if k in w and not w[k]["healthy"]]
        for k in dead:
            self.engines[k].state = EngineState.FAILED
            self._dispose(k, keep_record=True)
        return dead


@dataclass
class Rule:
    metric: str
    threshold: float
    direction: str            # "above" -> scale out, "below" -> scale in
    for_s: float = 30.0       # the condition must hold this long
    step: int = 1


@dataclass
class AutoscalerConfig:
    min_engines: int = 1
    max_engines: int = 8
    scale_out_cooldown_s: float = 120.0
    scale_in_cooldown_s: float = 300.0
    rules: List[Rule] = field(default_factory=lambda: [Rule("queue_depth_per_engine", 8.0, "above", 30.0),
                                                      Rule("kv_cache_utilization", 0.3, "below", 300.0)])

    @staticmethod
    def from_dict(d: dict) -> "AutoscalerConfig":
        rules = [Rule(**r) for r in d.get("rules", [])]
        kw = {k: v for k, v in d.items() if k != "rules"}
        return AutoscalerConfig(rules=rules or AutoscalerConfig().rules, **kw)


class Autoscaler:
    def __init__(self, pool: EnginePool, cfg: AutoscalerConfig, metrics_fn: Callable[[], Dict[str, float]],
                 clock: Callable[[], float] = time.monotonic):
        self.pool, self.cfg, self.metrics_fn, self.clock = pool, cfg, metrics_fn, clock
        self._since: Dict[int, Optional[float]] = {}
        self._last_out = self._last_in = -1e18
        self.decisions: list = []

    def step(self) -> Optional[str]:
        """Evaluate the rules once; returns ``"scale_out"``, ``"scale_in"`` or None."""
        now, m = self.clock(), self.metrics_fn()
        n = len(self.pool.active())
        action = None
        for i, r in enumerate(self.cfg.rules):
            v = m.get(r.metric)
            hit = v is not None and (v > r.threshold if r.direction == "above" else v < r.threshold)
            if not hit:
                self._since[i] = None
                continue
            if self._since.get(i) is None:
                self._since[i] = now
            if now - self._since[i] < r.for_s:
                continue
            if r.direction == "above" and n < self.cfg.max_engines and now - self._last_out >= self.cfg.scale_out_cooldown_s:
                k = min(r.step, self.cfg.max_engines - n)
                res = self.pool.scale_out(k)
                self._last_out, action = now, "scale_out"
                self.decisions.append((now, "scale_out", r.metric, v, list(res.succeeded)))
                self._since[i] = None
                break
            if (r.direction == "below" and n > self.cfg.min_engines and now - self._last_in >= self.cfg.scale_in_cooldown_s
                    and now - self._last_out >= self.cfg.scale_out_cooldown_s):
                removed = self.pool.scale_in(min(r.step, n - self.cfg.min_engines), min_engines=self.cfg.min_engines)
                self._last_in, action = now, "scale_in"
                self.decisions.append((now, "scale_in", r.metric, v, removed))
                self._since[i] = None
                break
        return action
