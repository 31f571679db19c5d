"""Inference permits: one permit = one model request in flight at the rollout engines.

Covers relax/engine/rollout/request_permit.py (``InferencePermitManager``, ``GenerationAborted``) and its
scheduling micro-benchmark (scripts/benchmarks/benchmark_request_permit.py).  Tool calls, environment steps and
tokenisation of a multi-turn session run *outside* the permit, so a long session does not hold a slot while it is
not talking to the engine.  The capacity follows the fleet: ``concurrency_per_engine * engines``, changed by
:meth:`resize` when the elastic pool scales out or in.

Works from threads (``with mgr.permit():``) and from asyncio (``async with mgr.apermit():``); neither form is
reentrant.

    python -m relax_b200.rollout.request_permit --sessions 256 --turns 4 --capacity 32     # the micro-benchmark
"""
from __future__ import annotations

import argparse
import asyncio
import threading
import time
from contextlib import asynccontextmanager, contextmanager
from typing import Callable, Optional


class GenerationAborted(Exception):
    """The rollout was aborted while the request waited for (or had just got) its permit."""


def capacity_for(concurrency_per_engine: int, rollout_gpus: int, gpus_per_engine: int) -> int:
    cap = concurrency_per_engine * rollout_gpus // max(1, gpus_per_engine)
    if cap < 1:
        raise ValueError(f"permit capacity {cap} < 1 (concurrency {concurrency_per_engine}, {rollout_gpus} GPUs, "
                         f"{gpus_per_engine} per engine): every request would block forever")
    return cap


class InferencePermitManager:
    def __init__(self, capacity: int):
        if capacity < 1:
            raise ValueError(f"capacity must be >= 1, got {capacity}")
        self.capacity = capacity
        self._in_use = 0
        self._cv = threading.Condition()
        self.peak = 0
        self.granted = 0

    # ------------------------------------------------------------------ core
    def acquire(self, abort_check: Optional[Callable[[], bool]] = None, timeout_s: Optional[float] = None) -> None:
        end = None if timeout_s is None else time.monotonic() + timeout_s
        with self._cv:
            while self._in_use >= self.capacity:
                if abort_check is not None and abort_check():
                    raise GenerationAborted()
                left = None if end is None else end - time.monotonic()
                if left is not None and left <= 0:
                    raise TimeoutError("no inference permit within the time limit")
                self._cv.wait(0.05 if left is None else min(0.05, left))
            self._in_use += 1
            self.granted += 1
            self.peak = max(self.peak, self._in_use)
        if abort_check is not None and abort_check():
            self.release()
            raise GenerationAborted()

    def release(self) -> None:
        with self._cv:
            if self._in_use <= 0:
                raise RuntimeError("release without acquire")
            self._in_use -= 1
            self._cv.notify()

    def resize(self, capacity: int) -> None:
        """New capacity; shrinking never revokes permits already held, it only delays new ones."""
        if capacity < 1:
            raise ValueError("capacity must be >= 1")
        with self._cv:
            self.capacity = capacity
            self._cv.notify_all()

    @property
    def in_use(self) -> int:
        return self._in_use

    # ------------------------------------------------------------------ context managers
    @contextmanager
    def permit(self, abort_check=None, timeout_s=None):
        self.acquire(abort_check, timeout_s)
        try:
            yield
        finally:
            self.release()

    @asynccontextmanager
    async def apermit(self, abort_check=None, timeout_s=None):
        await asyncio.get_running_loop().run_in_executor(None, self.acquire, abort_check, timeout_s)
        try:
            yield
        finally:
            self.release()


def benchmark(sessions: int = 256, turns: int = 4, capacity: int = 32, model_ms: float = 2.0, tool_ms: float = 2.0,
              hold_over_tools: bool = False) -> dict:
    """Multi-turn sessions that alternate a model request and a tool call.  With per-request permits the tool
    time overlaps other sessions' requests; holding the permit across the tool call (the naive session-level
    lock) serialises it."""
    mgr = InferencePermitManager(capacity)

    async def session():
        for _ in range(turns):
            if hold_over_tools:
                async with mgr.apermit():
                    await asyncio.sleep(model_ms / 1e3)
                    await asyncio.sleep(tool_ms / 1e3)
            else:
                async with mgr.apermit():
                    await asyncio.sleep(model_ms / 1e3)
                await asyncio.sleep(tool_ms / 1e3)

    async def run():
        loop = asyncio.get_running_loop()
        from concurrent.futures import ThreadPoolExecutor

        loop.set_default_executor(ThreadPoolExecutor(max_workers=max(64, 2 * capacity)))
        t0 = time.perf_counter()
        await asyncio.gather(*[session() for _ in range(sessions)])
        return time.perf_counter() - t0

    secs = asyncio.run(run())
    return {"seconds": secs, "requests_per_s": sessions * turns / secs, "peak_in_flight": mgr.peak, "granted": mgr.granted}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--sessions", type=int, default=256)
    ap.add_argument("--turns", type=int, default=4)
    ap.add_argument("--capacity", type=int, default=32)
    a = ap.parse_args()
    for hold in (False, True):
        print("hold permit over tool calls" if hold else "per-request permits", benchmark(a.sessions, a.turns, a.capacity, hold_over_tools=hold))
