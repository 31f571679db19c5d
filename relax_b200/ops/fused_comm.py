"""Fused compute + collective operators over NVLink peer memory.

Each function is the fused counterpart of an unfused ``torch.distributed`` + GEMM
pair in :mod:`relax_b200.parallel.tp` / :mod:`relax_b200.rollout.weights`.  A pair
is fused only for groups that were registered with :func:`attach` (which sets up
the symmetric buffers of :mod:`relax_b200.parallel.symm_mem`); otherwise callers
use the NCCL statement, which is also the A/B baseline.
"""
from __future__ import annotations

from typing import Optional

_ATTACHED: dict = {}


def attach(group_info, comm) -> None:
    """Register the symmetric-memory communicator of a process group."""
    _ATTACHED[tuple(group_info.ranks)] = comm


def detach(group_info) -> None:
    _ATTACHED.pop(tuple(group_info.ranks), None)


def comm_of(group_info) -> Optional[object]:
    return _ATTACHED.get(tuple(group_info.ranks))


def enabled_for(group_info) -> bool:
    return comm_of(group_info) is not None


def ag_gemm(x, w, g):
    return comm_of(g).ag_gemm(x, w)


def gemm_rs(x, w, g):
    return comm_of(g).gemm_rs(x, w)


def gemm_ar_add_rmsnorm(x, w, residual, norm_w, eps, g):
    return comm_of(g).gemm_ar_add_rmsnorm(x, w, residual, norm_w, eps)
