"""Row samplers for :meth:`TransferQueue.get_meta`.

A sampler is ``f(candidate_row_ids, custom_meta, batch_size) -> chosen_ids``.
``custom_meta`` carries ``total_lengths`` and ``sample_index`` per row
(relax/utils/utils.py:171-177).  Counterparts: the data-plane package's
``SeqlenBalancedSampler`` / ``StreamingTokenBudgetSampler`` and the in-tree
relax/utils/data/identity_window_sampler.py.
"""
from __future__ import annotations

from typing import Sequence

from .seqlen_balancing import karmarkar_karp


class SequentialSampler:
    def __call__(self, ready, meta, n):
        return ready[:n]


class SeqlenBalancedSampler:
    """Among the rows not yet taken by this task pick, for data-parallel replica
    ``dp_rank`` of ``dp_size``, the bin of a balanced ``dp_size``-way split of the
    first ``n * dp_size`` ready rows, so replicas get near-equal token counts."""

    def __init__(self, dp_rank: int = 0, dp_size: int = 1):
        self.dp_rank, self.dp_size = dp_rank, dp_size

    def __call__(self, ready, meta, n):
        if self.dp_size == 1:
            return ready[:n]
        window = ready[: n * self.dp_size]
        lens = [int(m.get("total_lengths", 1)) for m in meta[: len(window)]]
        if len(window) % self.dp_size:
            return window[self.dp_rank::self.dp_size][:n]
        bins = karmarkar_karp(lens, self.dp_size, equal_size=True)
        return [window[i] for i in bins[self.dp_rank]]


class StreamingTokenBudgetSampler:
    """Take ready rows in arrival order until the token budget is hit (at least
    one row); used by the fully-async trainer, which consumes while the rollout
    is still producing."""

    def __init__(self, max_tokens: int):
        self.max_tokens = max_tokens

    def __call__(self, ready, meta, n):
        out, tot = [], 0
        for rid, m in zip(ready, meta):
            L = int(m.get("total_lengths", 1))
            if out and tot + L > self.max_tokens:
                break
            out.append(rid)
            tot += L
            if n and len(out) >= n:
                break
        return out


class IdentityWindowSampler(StreamingTokenBudgetSampler):
    """Token-budget sampler that never splits the rows of one logical sample
    (multi-turn samples expand to several rows sharing ``sample_index``) and
    only hands out rows of the current window of ``window_samples`` logical
    samples, so an optimizer step sees a fixed set of samples regardless of
    arrival order."""

    def __init__(self, max_tokens: int, window_samples: int):
        super().__init__(max_tokens)
        self.window_samples = window_samples
        self.window_index = 0

    def advance_window(self):
        self.window_index += 1

    def __call__(self, ready, meta, n):
        lo = self.window_index * self.window_samples
        hi = lo + self.window_samples
        groups: dict = {}
        for rid, m in zip(ready, meta):
            si = int(m.get("sample_index", rid))
            if lo <= si < hi:
                groups.setdefault(si, []).append((rid, int(m.get("total_lengths", 1))))
        out, tot = [], 0
        for si in sorted(groups):
            gl = sum(L for _, L in groups[si])
            if out and tot + gl > self.max_tokens:
                break
            out.extend(r for r, _ in groups[si])
            tot += gl
        return out


class StreamingTQIterator:
    """Micro-batches pulled from the transfer queue on demand, while the rollout is still producing
    (relax/utils/data/stream_dataloader.py StreamingTQIterator :1071-1250).

    ``next()`` blocks until a token-budget-sized micro-batch of rows with all ``data_fields`` is available and returns
    ``(batch, meta)`` with ``__loss_scale__`` added to the batch; it stops when the partition is sealed and this task has
    consumed every row.  Rows of this data-parallel rank only: row ``i`` of the partition belongs to rank ``i % dp_size``
    (every rank sees the same partition, the rule keeps the ranks disjoint without talking to each other).  ``window_quota``
    bounds how many rows one iterator hands out (one optimizer window of a longer rollout)."""

    def __init__(self, queue, data_fields, partition_id: str, token_budget: int, loss_scale: float = 1.0, dp_rank: int = 0,
                 dp_size: int = 1, task_name: str = "actor_train", window_quota: int = 0, poll_s: float = 0.05,
                 timeout_s: float = 3600.0):
        self.q, self.fields, self.part, self.task = queue, list(data_fields), partition_id, f"{task_name}/dp{dp_rank}"
        self.loss_scale, self.dp_rank, self.dp_size = loss_scale, dp_rank, dp_size
        self.window_quota, self.poll_s, self.timeout_s = window_quota, poll_s, timeout_s
        self.handed_out = 0
        self._budget = StreamingTokenBudgetSampler(token_budget)

    def _sampler(self, ready, meta, n):
        mine = [(r, m) for r, m in zip(ready, meta) if int(r) % self.dp_size == self.dp_rank]
        if not mine:
            return []
        left = self.window_quota - self.handed_out if self.window_quota else 0
        return self._budget([r for r, _ in mine], [m for _, m in mine], left if self.window_quota else 0)

    def _mine_left(self) -> bool:
        """Rows of this rank that the task has not consumed yet (known only once the partition is sealed)."""
        with self.q._cv:
            part = self.q._p.get(self.part)
            if part is None:
                return True
            done = part.consumed.get(self.task, set())
            return any(int(r) % self.dp_size == self.dp_rank and r not in done for r in part.rows)

    def __iter__(self):
        return self

    def __next__(self):
        import time

        if self.window_quota and self.handed_out >= self.window_quota:
            raise StopIteration
        t0 = time.monotonic()
        while True:
            meta = self.q.get_meta(self.fields, 1, self.part, self.task, sampler=self._sampler, timeout=self.poll_s, allow_partial=True)
            if meta is not None and len(meta):
                self.handed_out += len(meta)
                batch = self.q.get_data(meta)
                batch["__loss_scale__"] = self.loss_scale
                return batch, meta
            with self.q._cv:
                part = self.q._p.get(self.part)
                sealed = part is not None and part.sealed
            if sealed and not self._mine_left():
                raise StopIteration
            if time.monotonic() - t0 > self.timeout_s:
                raise TimeoutError(f"no micro-batch from partition {self.part} within {self.timeout_s:.0f} s")
