"""Structured logging for multi-process runs: one configuration call per process, rank- and role-tagged records,
optional JSON lines, and a helper that logs a repeating message only every so often.

Covers relax/utils/logging_utils.py (logger setup, rank filter) in the form this framework's one-process-per-GPU
layout needs: every record carries ``rank`` and ``role``; by default only rank 0 logs at INFO while the other ranks
log warnings and errors, so that an 8-GPU job prints one copy of the progress lines but all of the problems.
"""
from __future__ import annotations

import json
import logging
import os
import sys
import time
from typing import Dict, Optional

_CONFIGURED = False


class _Context(logging.Filter):
    def __init__(self, rank: int, role: str):
        super().__init__()
        self.rank, self.role = rank, role

    def filter(self, record: logging.LogRecord) -> bool:
        record.rank, record.role = self.rank, self.role
        return True


class JsonFormatter(logging.Formatter):
    def format(self, record: logging.LogRecord) -> str:
        d = {"t": round(record.created, 3), "level": record.levelname, "rank": getattr(record, "rank", 0),
             "role": getattr(record, "role", ""), "logger": record.name, "msg": record.getMessage()}
        extra = getattr(record, "fields", None)
        if isinstance(extra, dict):
            d.update(extra)
        if record.exc_info:
            d["exc"] = self.formatException(record.exc_info)
        return json.dumps(d, default=str)


def configure_logging(role: str = "", rank: Optional[int] = None, level: Optional[str] = None, json_lines: Optional[bool] = None,
                      all_ranks: Optional[bool] = None, stream=None, force: bool = False) -> logging.Logger:
    """Set up the ``relax_b200`` logger tree.  Environment overrides: ``RELAX_B200_LOG_LEVEL``,
    ``RELAX_B200_LOG_JSON=1``, ``RELAX_B200_LOG_ALL_RANKS=1``."""
    global _CONFIGURED
    root = logging.getLogger("relax_b200")
    if _CONFIGURED and not force:
        return root
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    level = (level or os.environ.get("RELAX_B200_LOG_LEVEL", "INFO")).upper()
    json_lines = os.environ.get("RELAX_B200_LOG_JSON", "0") == "1" if json_lines is None else json_lines
    all_ranks = os.environ.get("RELAX_B200_LOG_ALL_RANKS", "0") == "1" if all_ranks is None else all_ranks
    for h in list(root.handlers):
        root.removeHandler(h)
    h = logging.StreamHandler(stream or sys.stderr)
    h.addFilter(_Context(rank, role))
    h.setFormatter(JsonFormatter() if json_lines else
                   logging.Formatter("%(asctime)s %(levelname).1s [%(role)s r%(rank)d] %(name)s: %(message)s", "%H:%M:%S"))
    root.addHandler(h)
    root.propagate = False
    eff = getattr(logging, level, logging.INFO)
    root.setLevel(eff if (rank == 0 or all_ranks) else max(eff, logging.WARNING))
    _CONFIGURED = True
    return root


def get_logger(name: str) -> logging.Logger:
    return logging.getLogger(name if name.startswith("relax_b200") else f"relax_b200.{name}")


def log_fields(logger: logging.Logger, level: int, msg: str, **fields) -> None:
    """A record with machine-readable fields (kept as keys in JSON mode, appended as ``k=v`` otherwise)."""
    if not logger.isEnabledFor(level):
        return
    text = msg if not fields else msg + " " + " ".join(f"{k}={v}" for k, v in fields.items())
    logger.log(level, text if not _json_mode(logger) else msg, extra={"fields": fields})


def _json_mode(logger: logging.Logger) -> bool:
    lg = logger
    while lg is not None:
        for h in lg.handlers:
            if isinstance(h.formatter, JsonFormatter):
                return True
        if not lg.propagate:
            break
        lg = lg.parent
    return False


class EveryN:
    """``if every("kv-full", 30): log.warning(...)``: true at most once per ``seconds`` per key, and reports how
    many calls were swallowed in between."""

    def __init__(self):
        self._last: Dict[str, float] = {}
        self._skipped: Dict[str, int] = {}

    def __call__(self, key: str, seconds: float) -> bool:
        now = time.monotonic()
        if now - self._last.get(key, -1e18) >= seconds:
            self._last[key] = now
            return True
        self._skipped[key] = self._skipped.get(key, 0) + 1
        return False

    def take_skipped(self, key: str) -> int:
        return self._skipped.pop(key, 0)
