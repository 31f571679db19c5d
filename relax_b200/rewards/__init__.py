"""Reward functions and their registry.

``async_rm(args, sample)`` / ``batched_async_rm(args, samples)`` mirror the
entry points of relax/engine/rewards/__init__.py; rule-based scorers live in
sibling modules and register themselves under the ``--rm-type`` names the
reference accepts (relax/engine/rewards/registry.py).
"""
from __future__ import annotations

import asyncio
import importlib
import inspect
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from typing import Callable, Optional, Sequence

from ..types import Sample


@dataclass
class RewardSpec:
    name: str
    fn: Callable            # fn(sample) -> float | dict   (sync or async)
    batched: bool = False   # fn(samples) -> list
    note: str = ""


_REGISTRY: dict[str, RewardSpec] = {}


def register_reward(name: str, fn: Callable = None, *, batched: bool = False, note: str = ""):
    def deco(f):
        _REGISTRY[name] = RewardSpec(name, f, batched, note)
        return f

    return deco(fn) if fn is not None else deco


def get_reward_spec(name: str) -> RewardSpec:
    _ensure_builtin()
    if name not in _REGISTRY:
        raise KeyError(f"unknown rm_type {name!r}; known: {list_reward_types()}")
    return _REGISTRY[name]


def list_reward_types() -> list:
    _ensure_builtin()
    return sorted(_REGISTRY)


_LOADED = False


def _ensure_builtin():
    global _LOADED
    if _LOADED:
        return
    _LOADED = True
    from . import rules  # noqa: F401  (registers on import)


def load_function(path: str) -> Callable:
    """``pkg.module.func`` or ``pkg.module:func`` -> callable."""
    mod, _, name = path.replace(":", ".").rpartition(".")
    return getattr(importlib.import_module(mod), name)


class RewardExecutionError(RuntimeError):
    pass


_POOL: Optional[ThreadPoolExecutor] = None


def _pool(workers: int = 8) -> ThreadPoolExecutor:
    global _POOL
    if _POOL is None:
        _POOL = ThreadPoolExecutor(max_workers=workers, thread_name_prefix="reward")
    return _POOL


async def async_rm(args, sample: Sample):
    """Score one sample; ``args.custom_rm_path`` overrides ``args.rm_type``."""
    custom = getattr(args, "custom_rm_path", None)
    fn = load_function(custom) if custom else get_reward_spec(getattr(args, "rm_type", "parity")).fn
    try:
        if inspect.iscoroutinefunction(fn):
            return await (fn(args, sample) if custom else fn(sample))
        loop = asyncio.get_running_loop()
        return await loop.run_in_executor(_pool(), (lambda: fn(args, sample)) if custom else (lambda: fn(sample)))
    except Exception as e:  # noqa: BLE001
        raise RewardExecutionError(f"reward failed for sample {sample.index}: {e!r}") from e


async def batched_async_rm(args, samples: Sequence[Sample]) -> list:
    custom = getattr(args, "custom_rm_path", None)
    if custom:
        fn = load_function(custom)
        if getattr(args, "group_rm", False):
            r = fn(args, list(samples))
            return await r if inspect.isawaitable(r) else r
    else:
        spec = get_reward_spec(getattr(args, "rm_type", "parity"))
        if spec.batched:
            return list(spec.fn(list(samples)))
    return list(await asyncio.gather(*[async_rm(args, s) for s in samples]))


def compute_rewards(args, samples: Sequence[Sample]) -> list:
    """Synchronous convenience wrapper."""
    try:
        asyncio.get_running_loop()
    except RuntimeError:
        return asyncio.run(batched_async_rm(args, samples))
    spec = get_reward_spec(getattr(args, "rm_type", "parity"))
    return [spec.fn(s) for s in samples]
