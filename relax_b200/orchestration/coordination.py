"""Barriers between roles that share GPUs: wait until the rollout engine has given its memory back, and wait until
the peers of a round have finished it.

Covers relax/distributed/coordination.py (``RolloutOffloadBarrier`` :28-47, ``PeerStepBarrier`` :50-122).  Roles in
this framework are threads or processes that expose plain callables (``status()`` / ``get_step()``), so the
barriers poll callables; every wait takes a deadline, because a peer that died must surface as an error on the
host rather than as a hang.
"""
from __future__ import annotations

import logging
import time
from typing import Callable, Dict, List, Optional, Tuple


class BarrierTimeout(TimeoutError):
    pass


class RolloutOffloadBarrier:
    """Blocks the trainer until the rollout side reports anything but ``"onload"``."""

    def __init__(self, get_status: Callable[[], str], poll_interval: float = 0.05, logger: Optional[logging.Logger] = None):
        self._get, self._poll, self._log = get_status, poll_interval, logger

    def wait_offloaded(self, timeout_s: float = 600.0) -> float:
        t0 = time.monotonic()
        while self._get() == "onload":
            if time.monotonic() - t0 > timeout_s:
                raise BarrierTimeout(f"rollout engine still holds its memory after {timeout_s:.0f} s")
            time.sleep(self._poll)
        return time.monotonic() - t0


class PeerStepBarrier:
    """A peer whose ``get_step()`` is strictly greater than ``round_id`` has finished every part of that round
    (backward, optimizer step, sleep) and released the GPUs it shares with the caller."""

    def __init__(self, peers: Dict[str, Callable[[], int]], poll_interval: float = 0.05, log_every: int = 200,
                 logger: Optional[logging.Logger] = None):
        self._peers, self._poll, self._every, self._log = dict(peers), poll_interval, max(1, log_every), logger

    def is_empty(self) -> bool:
        return not self._peers

    def list_pending(self, round_id: int) -> List[Tuple[str, int]]:
        out = []
        for role, get_step in self._peers.items():
            s = int(get_step())
            if s <= round_id:
                out.append((role, s))
        return out

    def wait_completed_round(self, round_id: int, timeout_s: float = 3600.0) -> int:
        t0, polls = time.monotonic(), 0
        while True:
            pending = self.list_pending(round_id)
            if not pending:
                return polls
            if self._log is not None and polls % self._every == 0:
                self._log.info("waiting on peers to finish round %d: %s", round_id,
                               ", ".join(f"{r}(step={s})" for r, s in pending))
            if time.monotonic() - t0 > timeout_s:
                raise BarrierTimeout(f"peers {pending} did not finish round {round_id} within {timeout_s:.0f} s")
            polls += 1
            time.sleep(self._poll)
