"""Tensor/sequence-parallel linear layers as autograd functions.

Two communication patterns exist per transformer block (sequence parallel):
``all-gather -> column-parallel GEMM`` and ``row-parallel GEMM -> reduce-scatter``.
On CUDA each pair is ONE fused kernel over NVLink peer memory
(:mod:`relax_b200.ops.fused_comm`); this file holds the unfused
``torch.distributed`` + GEMM statement used on CPU/gloo, as the A/B baseline,
and as the backward of the fused forward where no fused backward exists yet.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import ops
from .state import GroupInfo


def _ag(x, g: GroupInfo):
    if g.size == 1:
        return x
    out = torch.empty((x.shape[0] * g.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=g.group)
    return out


def _rs(x, g: GroupInfo):
    if g.size == 1:
        return x
    out = torch.empty((x.shape[0] // g.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x.contiguous(), group=g.group)
    return out


def _ar(x, g: GroupInfo):
    if g.size > 1:
        dist.all_reduce(x, group=g.group)
    return x


def _fused_enabled(x, g=None, op: str = "") -> bool:
    """Whether ``op`` runs as one fused kernel for group ``g``: CUDA tensors, a symmetric-memory
    communicator attached to the group that implements the operator, and not switched off."""
    if not (x.is_cuda and os.environ.get("RELAX_B200_FORCE_REFERENCE", "0") != "1" and
            os.environ.get("RELAX_B200_FUSED_TP", "1") == "1"):
        return False
    from ..ops import fused_comm

    comm = fused_comm.comm_of(g) if g is not None else None
    return comm is not None and comm.supports(op)


def _rs_of_product(x, w, g: GroupInfo, w_is_kn: bool):
    """reduce_scatter(x @ w.T) (or x @ w when ``w_is_kn``): fused over peer memory when available."""
    if g.size > 1 and _fused_enabled(x, g, "gemm_rs") and x.shape[0] % (g.size * 128) == 0:
        from ..ops import fused_comm

        comm = fused_comm.comm_of(g)
        n = w.shape[1] if w_is_kn else w.shape[0]
        if comm.fits_rs(x.shape[0], n):
            return comm.gemm_rs(x.contiguous(), w, w_is_kn)
    return _rs(ops.dgrad(x, w) if w_is_kn else ops.linear(x, w), g)


class _AGLinear(torch.autograd.Function):
    """y = all_gather(x_shard) @ w.T   (w is a column-parallel shard)."""

    @staticmethod
    def forward(ctx, x, w, g):
        ctx.g = g
        comm = None
        if g.size > 1 and _fused_enabled(x, g, "ag_gemm"):
            from ..ops import fused_comm

            comm = fused_comm.comm_of(g)
            if not (comm.fits_ag(x.shape[0], x.shape[1]) and w.shape[0] % 64 == 0 and w.stride(1) == 1):
                comm = None
        if comm is not None:
            y, _ = comm.ag_gemm(x, w)
        else:
            xf = _ag(x, g)
            y = ops.linear(xf, w)
        ctx.save_for_backward(x, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        g = ctx.g
        dy = dy.contiguous()
        xf = _ag(x, g)  # re-gather instead of keeping T*tp activations alive
        dx = _rs_of_product(dy, w, g, True)
        dw = ops.wgrad(dy, xf, w)
        return dx, dw, None


class _LinearRS(torch.autograd.Function):
    """y_shard = reduce_scatter(x @ w.T)   (w is a row-parallel shard)."""

    @staticmethod
    def forward(ctx, x, w, g):
        ctx.g = g
        ctx.save_for_backward(x, w)
        return _rs_of_product(x, w, g, False)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        g = ctx.g
        dyf = _ag(dy.contiguous(), g)
        dx = ops.dgrad(dyf, w)
        dw = ops.wgrad(dyf, x, w)
        return dx, dw, None


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g):
        ctx.g = g
        return x

    @staticmethod
    def backward(ctx, dy):
        return _ar(dy.contiguous().clone(), ctx.g), None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g):
        return _ar(x.contiguous().clone(), g)

    @staticmethod
    def backward(ctx, dy):
        return dy, None


class _GatherSeq(torch.autograd.Function):
    """all-gather along tokens forward, reduce-scatter backward."""

    @staticmethod
    def forward(ctx, x, g):
        ctx.g = g
        return _ag(x, g)

    @staticmethod
    def backward(ctx, dy):
        return _rs(dy.contiguous(), ctx.g), None


class _ScatterSeq(torch.autograd.Function):
    """keep my token slice forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x, g):
        ctx.g = g
        n = x.shape[0] // g.size
        return x[g.rank * n : (g.rank + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, dy):
        return _ag(dy.contiguous(), ctx.g), None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g):
        ctx.g = g
        return _rs(x, g)

    @staticmethod
    def backward(ctx, dy):
        return _ag(dy.contiguous(), ctx.g), None


def ag_linear(x, w, g: GroupInfo):
    return _AGLinear.apply(x, w, g) if g.size > 1 else ops.linear(x, w)


def linear_rs(x, w, g: GroupInfo):
    return _LinearRS.apply(x, w, g) if g.size > 1 else ops.linear(x, w)


def copy_to_tp(x, g):
    return _CopyToTP.apply(x, g) if g.size > 1 else x


def reduce_from_tp(x, g):
    return _ReduceFromTP.apply(x, g) if g.size > 1 else x


def gather_seq(x, g):
    return _GatherSeq.apply(x, g) if g.size > 1 else x


def scatter_seq(x, g):
    return _ScatterSeq.apply(x, g) if g.size > 1 else x


def reduce_scatter_seq(x, g):
    return _ReduceScatterSeq.apply(x, g) if g.size > 1 else x
