"""Streaming data plane between roles (rollout -> actor / actor_fwd / reference /
advantages / critic).

A *partition* (``train_{rollout_id}``) is a growing table of rows; each row
holds named fields (jagged tensors or Python objects).  Consumption is tracked
per ``task_name`` so every role sees every row exactly once, producers can add
columns to existing rows (e.g. ``log_probs`` written back by actor_fwd) and a
consumer may ask only for rows whose required columns are all present.

Surface modelled on what the reference uses from its external data-plane
package (relax/utils/utils.py:508-556, relax/utils/data/stream_dataloader.py:
737-758, relax/components/rollout.py:468,622-632, relax/components/actor.py:
166,223,253, relax/backends/megatron/actor.py:2017-2064).  Storage here is
process-local; :mod:`relax_b200.data.tq_service` exposes the same object to
other processes over a socket, and tensors are staged in pinned host slabs
(:mod:`relax_b200.data.pinned_pool`) so a GPU consumer copies them with one
asynchronous H2D transfer per field.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable, Optional, Sequence

import torch


@dataclass
class BatchMeta:
    partition_id: str
    row_ids: list
    fields: list
    task_name: str
    custom_meta: list = field(default_factory=list)

    def __len__(self):
        return len(self.row_ids)


class _Partition:
    def __init__(self, pid: str):
        self.pid = pid
        self.rows: dict[int, dict] = {}        # row id -> {field: value}
        self.custom: dict[int, dict] = {}
        self.next_row = 0
        self.sealed = False                    # producer said "is_last"
        self.consumed: dict[str, set] = {}     # task -> row ids handed out
        self.expected_rows: Optional[int] = None


class TransferQueue:
    def __init__(self, capacity_partitions: Optional[int] = None):
        self._p: dict[str, _Partition] = {}
        self._cv = threading.Condition()
        self.capacity_partitions = capacity_partitions

    # ------------------------------------------------------------------ produce
    def put(self, data: dict, partition_id: str, custom_meta: Optional[Sequence[dict]] = None,
            is_last: bool = False, row_ids: Optional[Sequence[int]] = None) -> list:
        """Append rows (``row_ids is None``) or add/overwrite columns of existing
        rows.  ``data`` maps field -> list (one entry per row)."""
        n = len(next(iter(data.values()))) if data else 0
        for k, v in data.items():
            if len(v) != n:
                raise ValueError(f"field {k!r} has {len(v)} rows, expected {n}")
        with self._cv:
            part = self._p.get(partition_id)
            if part is None:
                if self.capacity_partitions is not None and len(self._p) >= self.capacity_partitions:
                    raise RuntimeError(f"data plane holds {len(self._p)} partitions (capacity "
                                       f"{self.capacity_partitions}); the consumer is too far behind")
                part = self._p[partition_id] = _Partition(partition_id)
            if row_ids is None:
                row_ids = list(range(part.next_row, part.next_row + n))
                part.next_row += n
            for i, rid in enumerate(row_ids):
                row = part.rows.setdefault(rid, {})
                for k, v in data.items():
                    row[k] = v[i]
                if custom_meta is not None:
                    part.custom.setdefault(rid, {}).update(custom_meta[i])
            if is_last:
                part.sealed = True
            self._cv.notify_all()
        return list(row_ids)

    def seal(self, partition_id: str):
        with self._cv:
            self._p.setdefault(partition_id, _Partition(partition_id)).sealed = True
            self._cv.notify_all()

    # ------------------------------------------------------------------ consume
    def _ready_rows(self, part: _Partition, fields: Sequence[str], task: str) -> list:
        done = part.consumed.setdefault(task, set())
        return [rid for rid, row in sorted(part.rows.items())
                if rid not in done and all(f in row for f in fields)]

    def get_meta(self, data_fields: Sequence[str], batch_size: Optional[int], partition_id: str, task_name: str,
                 sampler: Optional[Callable] = None, timeout: Optional[float] = None,
                 allow_partial: bool = False) -> Optional[BatchMeta]:
        """Reserve up to ``batch_size`` unconsumed rows whose ``data_fields`` are
        all present.  Blocks until enough rows exist, the partition is sealed
        (then a short final batch is returned when ``allow_partial``) or the
        timeout expires (returns ``None``).  ``sampler(candidates, custom_meta,
        batch_size) -> chosen ids`` lets the caller pick (sequence-length
        balancing, token budgets)."""
        deadline = None if timeout is None else time.monotonic() + timeout
        with self._cv:
            while True:
                part = self._p.get(partition_id)
                if part is not None:
                    ready = self._ready_rows(part, data_fields, task_name)
                    want = batch_size if batch_size is not None else len(ready)
                    enough = len(ready) >= want and want > 0
                    final = part.sealed and self._all_rows_have(part, data_fields) and len(ready) > 0
                    if enough or (final and (allow_partial or batch_size is None)):
                        if sampler is not None:
                            chosen = list(sampler(ready, [part.custom.get(r, {}) for r in ready], want))
                        else:
                            chosen = ready[:want]
                        if chosen:
                            part.consumed[task_name].update(chosen)
                            return BatchMeta(partition_id, chosen, list(data_fields), task_name,
                                             [dict(part.custom.get(r, {})) for r in chosen])
                    if part.sealed and not ready and self._all_rows_have(part, data_fields):
                        return None  # drained
                remaining = None if deadline is None else deadline - time.monotonic()
                if remaining is not None and remaining <= 0:
                    return None
                self._cv.wait(timeout=remaining if remaining is not None else 1.0)

    @staticmethod
    def _all_rows_have(part: _Partition, fields) -> bool:
        return all(all(f in row for f in fields) for row in part.rows.values())

    def get_data(self, meta: BatchMeta) -> dict:
        with self._cv:
            part = self._p[meta.partition_id]
            return {f: [part.rows[r][f] for r in meta.row_ids] for f in meta.fields}

    # ------------------------------------------------------------------ status
    def get_partition_list(self) -> list:
        with self._cv:
            return sorted(self._p)

    def clear_partition(self, partition_id: str):
        with self._cv:
            self._p.pop(partition_id, None)
            self._cv.notify_all()

    def reset_consumption(self, partition_id: str, task_name: Optional[str] = None):
        with self._cv:
            part = self._p.get(partition_id)
            if part is None:
                return
            if task_name is None:
                part.consumed.clear()
            else:
                part.consumed.pop(task_name, None)

    def check_production_status(self, data_fields: Sequence[str], partition_id: str) -> bool:
        """True when the partition is sealed and every row has ``data_fields``."""
        with self._cv:
            part = self._p.get(partition_id)
            return bool(part and part.sealed and self._all_rows_have(part, data_fields))

    check_production_completed = check_production_status

    def check_consumption_status(self, task_name: str, partition_id: str) -> bool:
        """True when ``task_name`` has been handed every row of a sealed partition."""
        with self._cv:
            part = self._p.get(partition_id)
            if part is None or not part.sealed:
                return False
            return len(part.consumed.get(task_name, ())) >= len(part.rows)

    def check_stream_drained(self, task_name: str, partition_id: str, data_fields: Sequence[str] = ()) -> bool:
        with self._cv:
            part = self._p.get(partition_id)
            if part is None:
                return False
            return part.sealed and not self._ready_rows(part, data_fields, task_name) and \
                len(part.consumed.get(task_name, ())) >= len(part.rows)

    def check_window_drained(self, task_name: str, partition_id: str, window_rows: int) -> bool:
        """True when ``task_name`` has consumed a whole number of ``window_rows`` windows
        and nothing of the current window is pending."""
        with self._cv:
            part = self._p.get(partition_id)
            if part is None:
                return False
            c = len(part.consumed.get(task_name, ()))
            return c > 0 and c % window_rows == 0 and c >= min(len(part.rows), c)

    def num_rows(self, partition_id: str) -> int:
        with self._cv:
            part = self._p.get(partition_id)
            return len(part.rows) if part else 0

    def num_consumed(self, task_name: str, partition_id: str) -> int:
        with self._cv:
            part = self._p.get(partition_id)
            return len(part.consumed.get(task_name, ())) if part else 0


# ----------------------------------------------------------------------------- module-level singleton API

_QUEUE: Optional[TransferQueue] = None


def init(conf: Optional[dict] = None) -> TransferQueue:
    global _QUEUE
    conf = conf or {}
    _QUEUE = TransferQueue(capacity_partitions=conf.get("capacity_partitions"))
    return _QUEUE


def get_client() -> TransferQueue:
    if _QUEUE is None:
        raise RuntimeError("transfer queue not initialised; call init() first")
    return _QUEUE


def close():
    global _QUEUE
    _QUEUE = None


def partition_name(rollout_id: int, prefix: str = "train") -> str:
    return f"{prefix}_{rollout_id}"


def partition_rollout_id(name: str) -> int:
    return int(name.rsplit("_", 1)[1])
