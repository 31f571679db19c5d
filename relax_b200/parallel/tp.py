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


def _fused_enabled(x, g=None) -> bool:
    if not (x.is_cuda and os.environ.get("RELAX_B200_FORCE_REFERENCE", "0") != "1" and
            os.environ.get("RELAX_B200_FUSED_TP", "1") == "1"):
        return False
    from ..ops import fused_comm

    return g is not None and fused_comm.enabled_for(g)


class _AGLinear(torch.autograd.Function):
    """y = all_gather(x_shard) @ w.T   (w is a column-parallel shard)."""

    @staticmethod
    def forward(ctx, x, w, g):
        ctx.g = g
        if g.size > 1 and _fused_enabled(x, g):
            from ..ops import fused_comm

            y, xf = fused_comm.ag_gemm(x, w, g)
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
        dx = _rs(ops.dgrad(dy, w), g)
        dw = ops.wgrad(dy, xf, w)
        return dx, dw, None


class _LinearRS(torch.autograd.Function):
    """y_shard = reduce_scatter(x @ w.T)   (w is a row-parallel shard)."""

    @staticmethod
    def forward(ctx, x, w, g):
        ctx.g = g
        ctx.save_for_backward(x, w)
        if g.size > 1 and _fused_enabled(x, g):
            from ..ops import fused_comm

            return fused_comm.gemm_rs(x, w, g)
        return _rs(ops.linear(x, w), g)

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
