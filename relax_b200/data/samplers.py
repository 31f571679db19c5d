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
