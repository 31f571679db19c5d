"""Small agreement collectives used around streaming data and conditional branches.

* :func:`agree_drained` - every rank of the model-parallel groups must stop consuming a stream at the same
  micro-batch (relax/backends/megatron/collective_utils.py :31-33: all-reduce MIN over tp x cp, then pp).
* :class:`ConditionalBranchSync` - a branch that only some data-parallel ranks would run (the vision tower on a
  batch without images) is run by all or by none, so gradient reduction sees the same set of parameters on every
  rank (relax/backends/megatron/conditional_branch_sync.py :130: all-reduce MAX of an "active" flag).
* :func:`chunked_all_reduce` - all-reduce a large flat buffer in bounded pieces so that the transient NCCL
  staging stays small (relax/backends/megatron/megatron_patch/chunked_grad_coalesce_patch.py :120, 1 GiB default).
"""
from __future__ import annotations

from typing import Callable, Iterable, Optional

import torch
import torch.distributed as dist

from .state import GroupInfo


def _flag(value: bool, device) -> torch.Tensor:
    return torch.tensor([1 if value else 0], dtype=torch.int32, device=device)


def agree_drained(local_drained: bool, groups: Iterable[GroupInfo], device="cpu") -> bool:
    """True only when the stream is drained on every rank of every given group."""
    t = _flag(local_drained, device)
    for g in groups:
        if g is not None and g.size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=g.group)
    return bool(int(t))


class ConditionalBranchSync:
    def __init__(self, group: Optional[GroupInfo], device="cpu"):
        self.group, self.device = group, device
        self.calls = self.dummy_runs = 0

    def any_active(self, locally_active: bool) -> bool:
        t = _flag(locally_active, self.device)
        if self.group is not None and self.group.size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group.group)
        return bool(int(t))

    def run(self, locally_active: bool, branch: Callable[[], torch.Tensor], dummy: Callable[[], torch.Tensor]):
        """``branch()`` where this rank has input for it; ``dummy()`` (a forward on placeholder input whose result
        is multiplied by zero by the caller) where it has none but some other rank does; ``None`` when no rank has."""
        self.calls += 1
        if locally_active:
            self.any_active(True)
            return branch()
        if self.any_active(False):
            self.dummy_runs += 1
            return dummy() * 0.0
        return None


def chunked_all_reduce(flat: torch.Tensor, group: GroupInfo, chunk_bytes: int = 1 << 30, average: bool = False) -> int:
    """In-place sum (or mean) of ``flat`` over ``group`` in pieces of at most ``chunk_bytes``; returns the number of
    collectives issued."""
    if group is None or group.size == 1:
        return 0
    n = flat.numel()
    step = max(1, chunk_bytes // flat.element_size())
    calls = 0
    for lo in range(0, n, step):
        piece = flat[lo:lo + step]
        dist.all_reduce(piece, group=group.group)
        if average:
            piece.div_(group.size)
        calls += 1
    return calls
