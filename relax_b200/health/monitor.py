"""Health registry, checker thread, two-tier restart policy and the rollout-engine
health monitor.

Reference: ``HealthStatus`` / ``HealthChecker`` / ``HealthManager``
(relax/utils/health_system.py:38-481, 120 s heartbeat timeout, services beat every
10 s from relax/core/service.py:112-129), two-tier recovery in the controller
(relax/core/controller.py:977-1257: in-place restart for stateless roles, global
restart for actor / rollout / actor_fwd or after three in-place restarts, at most
``--max-global-restart`` global restarts), engine health polling
(relax/utils/health_monitor.py) and CI fault injection
(relax/distributed/ray/rollout.py:946-966).

All failure paths are driven from the host: a role raises, stops beating, or an
engine's ``health()`` callback reports failure / is forced unhealthy.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Optional

HEARTBEAT_TIMEOUT = 120.0
GLOBAL_RESTART_ROLES = ("actor", "rollout", "actor_fwd")
MAX_INPLACE_RESTARTS = 3


@dataclass
class ServiceHealthState:
    name: str
    last_beat: float = field(default_factory=time.monotonic)
    step: int = 0
    healthy: bool = True
    error: Optional[str] = None
    restart_count: int = 0
    registered_at: float = field(default_factory=time.monotonic)


class HealthRegistry:
    def __init__(self, heartbeat_timeout: float = HEARTBEAT_TIMEOUT, clock: Callable[[], float] = time.monotonic):
        self.timeout, self.clock = heartbeat_timeout, clock
        self._s: dict[str, ServiceHealthState] = {}
        self._lock = threading.Lock()

    def register(self, name: str):
        with self._lock:
            self._s[name] = ServiceHealthState(name, last_beat=self.clock(), registered_at=self.clock())

    def unregister(self, name: str):
        with self._lock:
            self._s.pop(name, None)

    def heartbeat(self, name: str, step: int = 0):
        with self._lock:
            st = self._s.get(name)
            if st is None:
                st = self._s[name] = ServiceHealthState(name, registered_at=self.clock())
            st.last_beat, st.step = self.clock(), step

    def report_error(self, name: str, error: str):
        with self._lock:
            st = self._s.setdefault(name, ServiceHealthState(name))
            st.healthy, st.error = False, error

    def mark_healthy(self, name: str):
        with self._lock:
            st = self._s.get(name)
            if st:
                st.healthy, st.error, st.last_beat = True, None, self.clock()

    def unhealthy(self) -> list[ServiceHealthState]:
        now = self.clock()
        with self._lock:
            return [s for s in self._s.values() if (not s.healthy) or (now - s.last_beat > self.timeout)]

    def status(self) -> dict:
        now = self.clock()
        with self._lock:
            return {n: {"healthy": s.healthy and now - s.last_beat <= self.timeout, "step": s.step, "error": s.error,
                        "since_beat": now - s.last_beat, "restarts": s.restart_count} for n, s in self._s.items()}

    def bump_restart(self, name: str) -> int:
        with self._lock:
            st = self._s.setdefault(name, ServiceHealthState(name))
            st.restart_count += 1
            return st.restart_count


def restart_tier(role: str, restart_count: int) -> str:
    """``inplace`` or ``global`` for a failed role."""
    if role in GLOBAL_RESTART_ROLES or restart_count >= MAX_INPLACE_RESTARTS:
        return "global"
    return "inplace"


class HealthManager:
    """Polls the registry (about once a second) and calls the restart hooks; gives up
    after ``max_global_restart`` global restarts by calling ``on_fatal``."""

    def __init__(self, registry: HealthRegistry, restart_inplace: Callable[[str], None],
                 restart_global: Callable[[str], None], on_fatal: Callable[[str], None],
                 max_global_restart: int = 3, interval: float = 1.0):
        self.reg, self.restart_inplace, self.restart_global, self.on_fatal = registry, restart_inplace, restart_global, on_fatal
        self.max_global, self.interval = max_global_restart, interval
        self.global_restarts = 0
        self._stop = threading.Event()
        self._t: Optional[threading.Thread] = None
        self.events: list = []

    def check_once(self):
        for st in self.reg.unhealthy():
            n = self.reg.bump_restart(st.name)
            tier = restart_tier(st.name, n - 1)
            self.events.append((st.name, tier, st.error or "heartbeat timeout"))
            if tier == "inplace":
                self.restart_inplace(st.name)
                self.reg.mark_healthy(st.name)
            else:
                if self.global_restarts >= self.max_global:
                    self.on_fatal(f"{st.name}: {st.error or 'heartbeat timeout'} after {self.global_restarts} global restarts")
                    self._stop.set()
                    return
                self.global_restarts += 1
                self.restart_global(st.name)
                for name in list(self.reg.status()):
                    self.reg.mark_healthy(name)
                return

    def start(self):
        def loop():
            while not self._stop.wait(self.interval):
                self.check_once()

        self._t = threading.Thread(target=loop, daemon=True, name="health-manager")
        self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join(2 * self.interval + 1)


class RolloutHealthMonitor:
    """Polls every engine's ``health()``; after ``max_failures`` consecutive failures the engine is
    handed to ``recover(engine_id)`` (kill + recreate; it gets weights at the next sync)."""

    def __init__(self, engines: dict, recover: Callable[[int], None], interval: float = 30.0, timeout: float = 30.0,
                 first_wait: float = 0.0, max_failures: int = 3):
        self.engines, self.recover = engines, recover
        self.interval, self.timeout, self.first_wait, self.max_failures = interval, timeout, first_wait, max_failures
        self.failures = {k: 0 for k in engines}
        self.forced_unhealthy: set = set()
        self.recovered: list = []

    def set_force_unhealthy(self, engine_id: int, flag: bool = True):
        (self.forced_unhealthy.add if flag else self.forced_unhealthy.discard)(engine_id)

    def poll_once(self):
        for eid, eng in list(self.engines.items()):
            ok = eid not in self.forced_unhealthy
            if ok:
                try:
                    ok = bool(eng.health())
                except Exception:  # noqa: BLE001
                    ok = False
            self.failures[eid] = 0 if ok else self.failures.get(eid, 0) + 1
            if self.failures[eid] >= self.max_failures:
                self.failures[eid] = 0
                self.forced_unhealthy.discard(eid)
                self.recover(eid)
                self.recovered.append(eid)


def maybe_inject_fault(ci_test: bool, use_fault_tolerance: bool, rollout_id: int, monitor: RolloutHealthMonitor,
                       engine_id: int = 0) -> bool:
    """CI fault injection: from rollout 2 on, mark one engine as crashed (host side only)."""
    if ci_test and use_fault_tolerance and rollout_id >= 2:
        monitor.set_force_unhealthy(engine_id)
        return True
    return False
