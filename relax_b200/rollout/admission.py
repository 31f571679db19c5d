"""Admission control for multi-turn (agentic) programs: token leases against the engines' KV capacity.

A multi-turn episode keeps growing its context over many engine calls; when too many episodes are in flight the KV
cache thrashes (requests wait for blocks, prefixes are evicted and recomputed).  The reference puts an admission
coordinator in front of its agentic pipeline (relax/agentic/session/admission.py: reservation = expanded prompt +
remaining completion budget, relax/agentic/session/admission_coordinator.py: FIFO waiters, ageing, a pressure guard
from the engines' KV gauges, a degraded bypass).  This is the same accounting for in-process engines:

* ``acquire(tokens)`` blocks until the lease fits: the sum of all leases stays below ``capacity_tokens`` and the engines'
  measured usage (``usage_fn() -> fraction``) stays below ``pressure_guard``.  Waiters are served first come, first
  served; one that has waited longer than ``max_wait_s`` is admitted anyway and the lease says so (``bypass``) - a slow
  episode is better than a stuck rollout.
* ``release(lease)`` returns the tokens and wakes the waiters.
* ``metrics()`` counts grants, bypasses, mean / max wait and the peak of reserved tokens.
"""
from __future__ import annotations

import itertools
import threading
import time
from collections import deque
from dataclasses import dataclass
from typing import Callable, Optional


def reservation_tokens(prompt_tokens: int, remaining_completion_tokens: int) -> int:
    """What an episode may still occupy: its context so far plus everything it may still generate."""
    return max(0, int(prompt_tokens)) + max(0, int(remaining_completion_tokens))


@dataclass(frozen=True)
class Lease:
    lease_id: int
    tokens: int
    bypass: bool          # admitted past the limits after waiting ``max_wait_s``
    waited_s: float


class AdmissionController:
    def __init__(self, capacity_tokens: int, pressure_guard: float = 0.95, max_wait_s: float = 120.0,
                 usage_fn: Optional[Callable[[], float]] = None, clock: Callable[[], float] = time.monotonic):
        if capacity_tokens <= 0:
            raise ValueError("capacity_tokens must be positive")
        self.capacity, self.guard, self.max_wait_s = int(capacity_tokens), float(pressure_guard), float(max_wait_s)
        self.usage_fn, self._clock = usage_fn, clock
        self._cv = threading.Condition()
        self._reserved = 0
        self._leases: dict = {}
        self._queue: deque = deque()          # tickets in arrival order
        self._ids = itertools.count(1)
        self._m = {"granted": 0, "bypassed": 0, "wait_sum_s": 0.0, "wait_max_s": 0.0, "peak_reserved": 0, "cancelled": 0}

    @classmethod
    def for_engine(cls, engine, headroom: float = 0.9, **kw) -> "AdmissionController":
        """Capacity and pressure from one in-process engine's block manager."""
        bm = engine.bm
        cap = int(bm.num_blocks * bm.block_size * headroom)
        return cls(cap, usage_fn=lambda: 1.0 - bm.num_free / max(1, bm.num_blocks), **kw)

    # ------------------------------------------------------------------ leases
    def _fits(self, tokens: int) -> bool:
        if self._reserved + tokens > self.capacity and self._reserved > 0:
            return False                      # a single oversized episode still runs, alone
        if self.usage_fn is not None and self._reserved > 0 and self.usage_fn() >= self.guard:
            return False
        return True

    def acquire(self, tokens: int, timeout_s: Optional[float] = None, cancelled: Optional[Callable[[], bool]] = None) -> Optional[Lease]:
        """Blocks until granted (or bypassed after ``max_wait_s``).  Returns None when ``timeout_s`` ran out or
        ``cancelled()`` became true while waiting."""
        tokens = max(0, int(tokens))
        t0 = self._clock()
        ticket = object()
        with self._cv:
            self._queue.append(ticket)
            try:
                while True:
                    waited = self._clock() - t0
                    head = self._queue[0] is ticket
                    aged = waited >= self.max_wait_s
                    if (head and self._fits(tokens)) or aged:
                        lease = Lease(next(self._ids), tokens, bypass=aged and not (head and self._fits(tokens)), waited_s=waited)
                        self._reserved += tokens
                        self._leases[lease.lease_id] = lease
                        m = self._m
                        m["granted"] += 1
                        m["bypassed"] += int(lease.bypass)
                        m["wait_sum_s"] += waited
                        m["wait_max_s"] = max(m["wait_max_s"], waited)
                        m["peak_reserved"] = max(m["peak_reserved"], self._reserved)
                        return lease
                    if (timeout_s is not None and waited >= timeout_s) or (cancelled is not None and cancelled()):
                        self._m["cancelled"] += 1
                        return None
                    left = self.max_wait_s - waited
                    if timeout_s is not None:
                        left = min(left, timeout_s - waited)
                    self._cv.wait(timeout=max(0.005, min(left, 0.25)))     # also re-reads the pressure gauge
            finally:
                try:
                    self._queue.remove(ticket)
                except ValueError:
                    pass
                self._cv.notify_all()

    def release(self, lease: Optional[Lease]):
        if lease is None:
            return
        with self._cv:
            if self._leases.pop(lease.lease_id, None) is not None:
                self._reserved = max(0, self._reserved - lease.tokens)
            self._cv.notify_all()

    def metrics(self, reset: bool = False) -> dict:
        with self._cv:
            m = dict(self._m)
            m.update(reserved=self._reserved, waiting=len(self._queue), capacity=self.capacity,
                     wait_mean_s=m["wait_sum_s"] / max(1, m["granted"]))
            if reset:
                for k in self._m:
                    self._m[k] = 0 if not isinstance(self._m[k], float) else 0.0
            return m
