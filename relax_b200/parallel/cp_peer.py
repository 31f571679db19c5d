"""Context parallelism with the KV exchange inside the attention kernels.

Ring attention moves K/V blocks between ranks with send/recv and runs one attention call per step.  On an
NVSwitch node every peer is one hop away at full bandwidth, so the exchange can be dropped altogether: each rank
publishes its K/V rows (forward) or its Q / dO / lse / delta rows (backward) in symmetric memory and the
flash-attention kernels of the other ranks read those tiles straight over NVLink with their TMA loads (no
multicast), tile by tile, while they compute.  In the backward pass the rank that owns a K/V chunk computes its
dK/dV against every rank's queries and adds the dQ contributions into the query owner's fp32 accumulator with
the kernel's ordinary global reductions, which work across NVLink.  The only other traffic is three small
barrier kernels on the ranks' signal pads.

Layout: zig-zag, as relax/backends/megatron/cp_utils.py:39-87 - rank ``r`` of ``cp`` holds chunks ``r`` and
``2cp-1-r`` of ``2cp`` equal chunks; a (query chunk ``a``, key chunk ``b``) pair is full attention when ``b < a``,
causal when ``b == a`` and empty otherwise.  Partial results of a query chunk are merged by their log-sum-exp.
The unfused statement is :func:`relax_b200.parallel.cp.ring_attention`.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .state import GroupInfo
from .symm_mem import SymmBuffer


def _C():
    from ..ops import cuda as C

    return C._load()


class CPComm:
    """Symmetric buffers of one context-parallel group for sequences of up to ``max_rows`` local rows."""

    def __init__(self, g: GroupInfo, device, max_rows: int, num_q_heads: int, num_kv_heads: int, head_dim: int = 128):
        assert head_dim == 128 and g.size <= 8
        self.g, self.device = g, torch.device(device)
        self.rows, self.hq, self.hkv, self.d = max_rows, num_q_heads, num_kv_heads, head_dim
        self.dev = self.device.index if self.device.index is not None else torch.cuda.current_device()
        kvb = 2 * max_rows * num_kv_heads * head_dim * 2
        qb = max_rows * num_q_heads * head_dim * 2
        self.kv = SymmBuffer(2 * kvb, g, self.device)          # two parities
        self.q = SymmBuffer(qb, g, self.device)
        self.do = SymmBuffer(qb, g, self.device)
        self.lse = SymmBuffer(num_q_heads * max_rows * 4, g, self.device)
        self.delta = SymmBuffer(num_q_heads * max_rows * 4, g, self.device)
        self.dq_acc = SymmBuffer(max_rows * num_q_heads * head_dim * 4, g, self.device)
        self.sig = SymmBuffer(1024, g, self.device)
        self.state = torch.zeros(16, dtype=torch.int32, device=self.device)
        self.wait_ns = int(os.environ.get("RELAX_B200_PEER_WAIT_MS", "5000")) * 1_000_000
        self.calls = 0
        torch.cuda.synchronize(self.device)
        import torch.distributed as dist

        dist.barrier(group=g.group)

    def view(self, buf: SymmBuffer, rank: int, shape, dtype, offset_bytes: int = 0) -> torch.Tensor:
        return _C().tensor_from_ptr(buf.ptrs[rank] + offset_bytes, list(shape), dtype, self.dev)

    def barrier(self, slot: int):
        from ..ops import cuda as C

        _C().peer_barrier(self.sig.ptrs, self.state, self.g.rank, slot, slot, self.wait_ns, C.err_flag(self.device))

    def close(self):
        for b in (self.kv, self.q, self.do, self.lse, self.delta, self.dq_acc, self.sig):
            b.close()


def _chunk_ids(rank: int, cp: int):
    return (rank, 2 * cp - 1 - rank)


def _valid(chunk: int, cs: int, total: int) -> int:
    return max(0, min(cs, total - chunk * cs))


def _cu(a0: int, n: int, device) -> torch.Tensor:
    return torch.tensor([a0, a0 + n], dtype=torch.int32, device=device)


class _PeerAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, comm: CPComm, total_length: int, scale: float):
        from ..ops import cuda as C

        g, cp, me = comm.g, comm.g.size, comm.g.rank
        rows, Hq, D = q.shape
        Hkv = k.shape[1]
        cs = rows // 2
        if rows > comm.rows or Hq != comm.hq or Hkv != comm.hkv:
            raise ValueError("sequence does not fit the context-parallel buffers")
        parity = comm.calls & 1
        comm.calls += 1
        kvb = 2 * comm.rows * Hkv * D * 2
        mine = comm.view(comm.kv, me, (2, rows, Hkv, D), q.dtype, parity * kvb)
        mine[0].copy_(k)
        mine[1].copy_(v)
        comm.barrier(0)
        q = q.contiguous()
        o_acc = torch.zeros(rows, Hq, D, dtype=torch.float32, device=q.device)
        lse_acc = torch.full((Hq, rows), float("-inf"), device=q.device)
        err = C.err_flag(q.device)
        for step in range(cp):
            s = (me + step) % cp                      # own chunks first, then the peers
            kv_s = comm.view(comm.kv, s, (2, rows, Hkv, D), q.dtype, parity * kvb)
            for bi, b in enumerate(_chunk_ids(s, cp)):
                kvn = _valid(b, cs, total_length)
                for ai, a in enumerate(_chunk_ids(me, cp)):
                    qn = _valid(a, cs, total_length)
                    if b > a or kvn == 0 or qn == 0:
                        continue
                    o_p = torch.empty(rows, Hq, D, dtype=q.dtype, device=q.device)
                    lse_p = torch.empty(Hq, rows, dtype=torch.float32, device=q.device)
                    _C().fa_fwd(q, kv_s[0], kv_s[1], o_p, lse_p, _cu(ai * cs, qn, q.device), _cu(bi * cs, kvn, q.device),
                                (qn + 127) // 128 + 1, b == a, scale, err)
                    r0, r1 = ai * cs, ai * cs + qn
                    new = torch.logaddexp(lse_acc[:, r0:r1], lse_p[:, r0:r1])
                    wa = torch.exp(lse_acc[:, r0:r1] - new).t().unsqueeze(-1)
                    wb = torch.exp(lse_p[:, r0:r1] - new).t().unsqueeze(-1)
                    o_acc[r0:r1] = o_acc[r0:r1] * wa + o_p[r0:r1].float() * wb
                    lse_acc[:, r0:r1] = new
        out = o_acc.to(q.dtype)
        ctx.save_for_backward(q, k.contiguous(), v.contiguous(), out, lse_acc)
        ctx.comm, ctx.total_length, ctx.scale = comm, total_length, scale
        return out

    @staticmethod
    def backward(ctx, do):
        from ..ops import cuda as C

        q, k, v, out, lse = ctx.saved_tensors
        comm, total, scale = ctx.comm, ctx.total_length, ctx.scale
        g, cp, me = comm.g, comm.g.size, comm.g.rank
        rows, Hq, D = q.shape
        Hkv = k.shape[1]
        cs = rows // 2
        do = do.contiguous()
        # publish what the owners of the K/V chunks need from me
        comm.view(comm.q, me, (rows, Hq, D), q.dtype).copy_(q)
        comm.view(comm.do, me, (rows, Hq, D), q.dtype).copy_(do)
        lse_pub = torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))
        comm.view(comm.lse, me, (Hq, rows), torch.float32).copy_(lse_pub)
        comm.view(comm.delta, me, (Hq, rows), torch.float32).copy_((out.float() * do.float()).sum(-1).t())
        my_acc = comm.view(comm.dq_acc, me, (rows, Hq, D), torch.float32)
        my_acc.zero_()
        comm.barrier(1)
        dk = torch.zeros(rows, Hkv, D, dtype=torch.float32, device=q.device)
        dv = torch.zeros_like(dk)
        err = C.err_flag(q.device)
        dummy = torch.empty(0, dtype=q.dtype, device=q.device)
        for step in range(cp):
            s = (me + step) % cp
            q_s = comm.view(comm.q, s, (rows, Hq, D), q.dtype)
            do_s = comm.view(comm.do, s, (rows, Hq, D), q.dtype)
            lse_s = comm.view(comm.lse, s, (Hq, rows), torch.float32)
            dl_s = comm.view(comm.delta, s, (Hq, rows), torch.float32)
            acc_s = comm.view(comm.dq_acc, s, (rows, Hq, D), torch.float32)
            for bi, b in enumerate(_chunk_ids(me, cp)):          # my K/V chunks
                kvn = _valid(b, cs, total)
                for ai, a in enumerate(_chunk_ids(s, cp)):       # the peer's query chunks
                    qn = _valid(a, cs, total)
                    if a < b or kvn == 0 or qn == 0:
                        continue
                    dk_p = torch.zeros(rows, Hkv, D, dtype=q.dtype, device=q.device)
                    dv_p = torch.zeros_like(dk_p)
                    _C().fa_bwd_ex(q_s, k, v, q_s, do_s, lse_s, dummy, dk_p, dv_p, dl_s, acc_s, _cu(ai * cs, qn, q.device),
                                   _cu(bi * cs, kvn, q.device), (kvn + 127) // 128 + 1, a == b, scale, 1 | 2 | 4, err)
                    dk += dk_p.float()
                    dv += dv_p.float()
        comm.barrier(2)                                          # every rank has added its share into my accumulator
        dq = torch.empty_like(q)
        _C().fa_dq_convert(my_acc, dq)
        return dq, dk.to(k.dtype), dv.to(v.dtype), None, None, None


def peer_attention(q, k, v, comm: CPComm, total_length: int, scale: Optional[float] = None):
    """Causal attention of one zig-zag-sharded sequence; ``q/k/v`` are this rank's two chunks (bf16, head_dim 128)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _PeerAttention.apply(q, k, v, comm, total_length, float(scale))
