"""Loading user code by path: custom generate functions, reward functions, filters, converters.

Covers relax/engine/rollout/forge_load.py (custom generate loader) and the ``--custom-generate-function-path`` /
``--custom-rm-path`` family of flags: a target is ``package.module:attr``, ``package.module.attr`` or
``/path/to/file.py:attr``.  Loaded callables are cached per path and their arity is checked when they are
loaded, so that a wrong path or signature fails at start-up and not in the middle of a rollout.
"""
from __future__ import annotations

import hashlib
import importlib
import importlib.util
import inspect
import os
import sys
from typing import Any, Callable, Optional

_CACHE: dict = {}


def load_object(path: str) -> Any:
    if path in _CACHE:
        return _CACHE[path]
    mod_part, sep, attr = path.rpartition(":")
    if not sep:
        mod_part, _, attr = path.rpartition(".")
    if not mod_part or not attr:
        raise ValueError(f"{path!r}: expected 'module:attr', 'module.attr' or 'file.py:attr'")
    if mod_part.endswith(".py") or os.sep in mod_part:
        if not os.path.isfile(mod_part):
            raise FileNotFoundError(mod_part)
        name = "relax_b200_user_" + hashlib.sha1(os.path.abspath(mod_part).encode()).hexdigest()[:12]
        mod = sys.modules.get(name)      # one module object per file, however many attributes are loaded from it
        if mod is None:
            spec = importlib.util.spec_from_file_location(name, mod_part)
            mod = importlib.util.module_from_spec(spec)
            sys.modules[name] = mod
            try:
                spec.loader.exec_module(mod)
            except BaseException:
                sys.modules.pop(name, None)
                raise
    else:
        mod = importlib.import_module(mod_part)
    obj = mod
    for part in attr.split("."):
        if not hasattr(obj, part):
            raise AttributeError(f"{mod_part!r} has no attribute {attr!r}")
        obj = getattr(obj, part)
    _CACHE[path] = obj
    return obj


def reload_object(path: str) -> Any:
    """Load ``path`` again from its source: the cached object is dropped and the module is re-executed (a user file is
    re-read from disk, an importable module goes through ``importlib.reload``).  For hot-reloading user code in a
    running job (relax/utils/reload_utils.py)."""
    _CACHE.pop(path, None)
    mod_part, sep, _ = path.rpartition(":")
    if not sep:
        mod_part, _, _ = path.rpartition(".")
    if mod_part.endswith(".py") or os.sep in mod_part:
        name = "relax_b200_user_" + hashlib.sha1(os.path.abspath(mod_part).encode()).hexdigest()[:12]
        sys.modules.pop(name, None)
        for k in [k for k in _CACHE if k.startswith(mod_part + ":")]:
            _CACHE.pop(k, None)               # other attributes of the same file were bound to the old module
    elif mod_part in sys.modules:
        importlib.reload(sys.modules[mod_part])
    return load_object(path)


def load_function(path: str, min_positional: int = 0, name: str = "function") -> Callable:
    """``load_object`` plus a check that the callable accepts at least ``min_positional`` positional arguments."""
    fn = load_object(path)
    if not callable(fn):
        raise TypeError(f"{name} {path!r} is not callable")
    try:
        sig = inspect.signature(fn)
    except (TypeError, ValueError):
        return fn
    params = list(sig.parameters.values())
    if any(p.kind is p.VAR_POSITIONAL for p in params):
        return fn
    npos = sum(1 for p in params if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD))
    if npos < min_positional:
        raise TypeError(f"{name} {path!r} takes {npos} positional arguments, needs at least {min_positional}")
    return fn


def load_generate_function(path: Optional[str], default: Callable) -> Callable:
    """The rollout's generate function: ``fn(engine, samples, sampling_params) -> samples``.  A function that sets
    ``manages_inference_permit = True`` takes and returns permits itself (multi-turn code that must not hold one
    over its tool calls); otherwise the caller wraps every call in a permit."""
    if not path:
        return default
    return load_function(path, 3, "generate function")


def manages_inference_permit(fn: Callable) -> bool:
    return bool(getattr(fn, "manages_inference_permit", False))
