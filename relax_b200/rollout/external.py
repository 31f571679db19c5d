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


class ExternalEngine:
    def __init__(self, cfg, addrs: Sequence[str], device, dtype, max_model_len: Optional[int] = None, timeout_s: float = 3600.0,
                 check_fields: Sequence[str] = ("model",)):
        from .weights import RolloutWeights

        if not addrs:
            raise ValueError("--rollout-external needs --rollout-external-engine-addrs")
        if cfg.vision is not None:
            raise NotImplementedError("image prompts do not travel over the HTTP surface: external engines serve text models")
        self.cfg, self.device, self.dtype, self.max_model_len = cfg, device, dtype, max_model_len
        self.clients = [HTTPEngine(a if "://" in a else f"http://{a}", timeout_s) for a in addrs]
        self.weights = RolloutWeights(cfg, 1, 0, device, dtype)          # staging, in the servers' layout (TP 1)
        self.weight_version = 0
        self.running: list = []
        self.paused = False
        self.bm = None                                                   # no local KV cache
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "cached_tokens": 0, "steps": 0}
        self._pool = ThreadPoolExecutor(max_workers=max(1, len(self.clients)), thread_name_prefix="ext-engine")
        self._lock = threading.Lock()
        for c in self.clients:
            info = c.info()
            for f in check_fields:
                want = {"model": cfg.name}.get(f)
                if want is not None and info.get(f) != want:
                    raise ValueError(f"{c.url} serves {f}={info.get(f)!r}, this job trains {want!r}")

    # ------------------------------------------------------------------ what WeightSync calls
    def _all(self, fn):
        return list(self._pool.map(fn, self.clients))

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
        """Prompt groups are kept together (prefix sharing on the server) and spread over the servers in contiguous
        runs; results come back in the order of ``prompts``."""
        if images is not None and any(images):
            raise NotImplementedError("image prompts do not travel over the HTTP surface")
        n, k = len(prompts), len(self.clients)
        keys = list(group_keys) if group_keys is not None else list(range(n))
        order = sorted(range(n), key=lambda i: (str(keys[i]), i))
        groups: list = []
        for i in order:
            if groups and keys[groups[-1][-1]] == keys[i]:
                groups[-1].append(i)
            else:
                groups.append([i])
        shares = [[] for _ in range(k)]
        for g_i, g in enumerate(groups):
            shares[g_i * k // max(1, len(groups))] += g
        out = [None] * n

        def run(j):
            idx = shares[j]
            if not idx:
                return
            sp = params if not isinstance(params, (list, tuple)) else params[idx[0]]
            for i, r in zip(idx, self.clients[j].generate([prompts[i] for i in idx], sp)):
                out[i] = r

        list(self._pool.map(run, range(k)))
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
