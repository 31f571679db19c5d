"""Typed registry of the environment variables the framework reads, with validation at start-up
(relax/utils/env.py ``EnvProperty`` / ``validate_env``): one place that says which variables
exist, their type, default and allowed values, so a typo in a launch script fails loudly.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Sequence


@dataclass
class EnvProperty:
    name: str
    type: Callable[[str], Any] = str
    default: Any = None
    choices: Optional[Sequence] = None
    doc: str = ""

    def get(self, environ=None):
        raw = (environ if environ is not None else os.environ).get(self.name)
        if raw is None:
            return self.default
        try:
            v = _to_bool(raw) if self.type is bool else self.type(raw)
        except ValueError as e:
            raise ValueError(f"environment variable {self.name}={raw!r} is not a valid {self.type.__name__}") from e
        if self.choices is not None and v not in self.choices:
            raise ValueError(f"environment variable {self.name}={raw!r} must be one of {list(self.choices)}")
        return v


def _to_bool(s: str) -> bool:
    if s.lower() in ("1", "true", "yes", "on"):
        return True
    if s.lower() in ("0", "false", "no", "off", ""):
        return False
    raise ValueError(s)


REGISTRY: Dict[str, EnvProperty] = {}


def register(name: str, type=str, default=None, choices=None, doc: str = "") -> EnvProperty:
    p = EnvProperty(name, type, default, choices, doc)
    REGISTRY[name] = p
    return p


FORCE_REFERENCE = register("RELAX_B200_FORCE_REFERENCE", bool, False, doc="run the PyTorch statements instead of the sm_100a kernels")
FUSED_TP = register("RELAX_B200_FUSED_TP", bool, True, doc="fuse TP GEMMs with their collectives over NVLink peer memory")
FUSED_LOCAL = register("RELAX_B200_FUSED_LOCAL", bool, False, doc="single-rank split-K GEMM + reduce + norm in one launch")
PEER_WAIT_MS = register("RELAX_B200_PEER_WAIT_MS", int, 5000, doc="limit of a kernel's wait for its NVLink peers")
DECODE_ATTN_VERSION = register("RELAX_B200_DECODE_ATTN_VERSION", int, 3, choices=(1, 2, 3), doc="paged decode attention kernel")
CRASH_TRACE = register("RELAX_B200_CRASH_TRACE", bool, False, doc="print a native backtrace on SIGSEGV/SIGABRT")
LOCAL_PLAN = register("RELAX_B200_LOCAL_PLAN", str, "splitk", choices=("splitk", "ar"))


def validate_env(environ=None, prefix: str = "RELAX_B200_") -> dict:
    """Parse every registered variable and reject unknown ones with the framework's prefix."""
    env = environ if environ is not None else os.environ
    unknown = [k for k in env if k.startswith(prefix) and k not in REGISTRY]
    if unknown:
        raise ValueError(f"unknown environment variable(s) {unknown}; known: {sorted(REGISTRY)}")
    return {k: p.get(env) for k, p in REGISTRY.items()}
