"""Partition sequences into k bins of near-equal total length.

``karmarkar_karp`` is the largest-differencing method on k-tuples (the
algorithm the reference uses in relax/utils/data/seqlen_balancing.py); bins can
be forced to equal cardinality.  ``first_fit_decreasing`` packs under a token
cap (used to form micro-batches for ``--use-dynamic-batch-size``).
"""
from __future__ import annotations

import heapq
from typing import Sequence


def karmarkar_karp(lengths: Sequence[int], k: int, equal_size: bool = False) -> list[list[int]]:
    """Return ``k`` lists of indices.  With ``equal_size`` every bin gets
    ``len(lengths) / k`` items (the count must divide)."""
    n = len(lengths)
    if k <= 0:
        raise ValueError("k must be positive")
    if equal_size and n % k:
        raise ValueError(f"{n} items do not split evenly into {k} bins")
    order = sorted(range(n), key=lambda i: lengths[i], reverse=True)
    # state: (neg spread, tie, [(sum, [idx...]) * k] sorted by sum desc)
    heap = []
    tie = 0
    if equal_size:
        for s in range(0, n, k):
            grp = order[s:s + k]
            bins = sorted(((lengths[i], [i]) for i in grp), key=lambda b: -b[0])
            heapq.heappush(heap, (-(bins[0][0] - bins[-1][0]), tie, bins))
            tie += 1
    else:
        for i in order:
            bins = [(lengths[i], [i])] + [(0, []) for _ in range(k - 1)]
            heapq.heappush(heap, (-lengths[i], tie, bins))
            tie += 1
    if not heap:
        return [[] for _ in range(k)]
    while len(heap) > 1:
        _, _, a = heapq.heappop(heap)
        _, _, b = heapq.heappop(heap)
        # combine largest of a with smallest of b
        merged = [(a[i][0] + b[k - 1 - i][0], a[i][1] + b[k - 1 - i][1]) for i in range(k)]
        merged.sort(key=lambda x: -x[0])
        heapq.heappush(heap, (-(merged[0][0] - merged[-1][0]), tie, merged))
        tie += 1
    return [sorted(b[1]) for b in heap[0][2]]


def first_fit_decreasing(lengths: Sequence[int], cap: int) -> list[list[int]]:
    """Bins of indices whose lengths sum to at most ``cap`` (items longer than
    the cap get a bin of their own)."""
    order = sorted(range(len(lengths)), key=lambda i: lengths[i], reverse=True)
    bins: list[list[int]] = []
    loads: list[int] = []
    for i in order:
        L = lengths[i]
        for b in range(len(bins)):
            if loads[b] + L <= cap:
                bins[b].append(i)
                loads[b] += L
                break
        else:
            bins.append([i])
            loads.append(L)
    return [sorted(b) for b in bins]


def balanced_microbatches(lengths: Sequence[int], cap: int, min_bins: int = 1, multiple_of: int = 1) -> list[list[int]]:
    """Choose the number of micro-batches from the token cap (at least
    ``min_bins``, rounded up to ``multiple_of`` - e.g. the pipeline's
    micro-batch group size) and balance their token totals."""
    need = max(min_bins, len(first_fit_decreasing(lengths, cap)))
    need = (need + multiple_of - 1) // multiple_of * multiple_of
    need = min(need, max(1, len(lengths))) if len(lengths) >= multiple_of else need
    while True:
        bins = karmarkar_karp(lengths, need)
        if all(sum(lengths[i] for i in b) <= cap or len(b) <= 1 for b in bins) or need >= len(lengths):
            return [b for b in bins]
        need += multiple_of
