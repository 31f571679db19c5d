"""Context parallelism over NVLink symmetric memory, without a ring.

Ring attention moves K/V blocks between ranks with send/recv and runs one attention call per step.  On an
NVSwitch node every peer is one hop away at full bandwidth, so each tensor crosses the links exactly once:
in the forward pass every rank pushes its K/V rows into a slot of every peer's staging buffer (peer stores from
one copy kernel), computes the attention of its own chunks while the peers' rows arrive, passes a barrier on the
signal pads, and then attends to the peers' chunks out of LOCAL memory.  The backward pass pushes Q / dO / lse /
delta the same way; the owner of a K/V chunk computes dK/dV against every rank's queries, accumulates the dQ
contributions for a peer's queries in a local fp32 buffer and pushes that buffer once into a slot on the
queries' owner, who sums the slots.  (Reading the peers' tiles directly from inside the attention kernels also
works - the kernels' TMA loads and global reductions are valid on peer mappings - but every query block would
pull the same K/V tile over NVLink again: 5.6x slower at 32k tokens than the ideal, so the data is staged.)

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
        n = g.size
        self.kv_slot = 2 * max_rows * num_kv_heads * head_dim * 2          # K and V of one rank
        self.q_slot = max_rows * num_q_heads * head_dim * 2
        self.st_slot = num_q_heads * max_rows * 4
        self.dq_slot = max_rows * num_q_heads * head_dim * 4
        # every buffer has one slot per source rank; K/V is double buffered by call parity
        self.kv = SymmBuffer(2 * n * self.kv_slot, g, self.device)
        self.q = SymmBuffer(n * self.q_slot, g, self.device)
        self.do = SymmBuffer(n * self.q_slot, g, self.device)
        self.lse = SymmBuffer(n * self.st_slot, g, self.device)
        self.delta = SymmBuffer(n * self.st_slot, g, self.device)
        self.dq_acc = SymmBuffer(n * self.dq_slot, g, self.device)
        self.sig = SymmBuffer(1024, g, self.device)
        self.state = torch.zeros(16, dtype=torch.int32, device=self.device)
        self.wait_ns = int(os.environ.get("RELAX_B200_PEER_WAIT_MS", "5000")) * 1_000_000
        self.calls = 0
        torch.cuda.synchronize(self.device)
        import torch.distributed as dist

        dist.barrier(group=g.group)

    def view(self, buf: SymmBuffer, rank: int, shape, dtype, offset_bytes: int = 0) -> torch.Tensor:
        return _C().tensor_from_ptr(buf.ptrs[rank] + offset_bytes, list(shape), dtype, self.dev)

    def push(self, src: torch.Tensor, buf: SymmBuffer, offset_bytes: int, ranks=None):
        """Copy ``src`` to ``offset_bytes`` of ``buf`` on the given ranks (default: every rank but this one)."""
        ranks = [r for r in range(self.g.size) if r != self.g.rank] if ranks is None else list(ranks)
        if ranks:
            _C().peer_push(src.contiguous(), [buf.ptrs[r] for r in ranks], offset_bytes)

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
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        half = comm.rows * Hkv * D * 2

        def region(src):
            return (parity * cp + src) * comm.kv_slot

        comm.push(k, comm.kv, region(me))
        comm.push(v, comm.kv, region(me) + half)
        o_acc = torch.zeros(rows, Hq, D, dtype=torch.float32, device=q.device)
        lse_acc = torch.full((Hq, rows), float("-inf"), device=q.device)
        err = C.err_flag(q.device)
        for step in range(cp):
            s = (me + step) % cp                      # own chunks first: the peers' rows arrive meanwhile
            if step == 1:
                comm.barrier(0)
            if s == me:
                k_s, v_s = k, v
            else:
                k_s = comm.view(comm.kv, me, (rows, Hkv, D), q.dtype, region(s))
                v_s = comm.view(comm.kv, me, (rows, Hkv, D), q.dtype, region(s) + half)
            for bi, b in enumerate(_chunk_ids(s, cp)):
                kvn = _valid(b, cs, total_length)
                for ai, a in enumerate(_chunk_ids(me, cp)):
                    qn = _valid(a, cs, total_length)
                    if b > a or kvn == 0 or qn == 0:
                        continue
                    o_p = torch.empty(rows, Hq, D, dtype=q.dtype, device=q.device)
                    lse_p = torch.empty(Hq, rows, dtype=torch.float32, device=q.device)
                    _C().fa_fwd(q, k_s, v_s, o_p, lse_p, _cu(ai * cs, qn, q.device), _cu(bi * cs, kvn, q.device),
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
        lse_pub = torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse)).contiguous()
        delta = (out.float() * do.float()).sum(-1).t().contiguous()
        # hand the owners of the other K/V chunks what they need from me (slot = my rank, in THEIR memory)
        comm.push(q, comm.q, me * comm.q_slot)
        comm.push(do, comm.do, me * comm.q_slot)
        comm.push(lse_pub, comm.lse, me * comm.st_slot)
        comm.push(delta, comm.delta, me * comm.st_slot)
        dk = torch.zeros(rows, Hkv, D, dtype=torch.float32, device=q.device)
        dv = torch.zeros_like(dk)
        dq_tot = torch.zeros(rows, Hq, D, dtype=torch.float32, device=q.device)
        err = C.err_flag(q.device)
        dummy = torch.empty(0, dtype=q.dtype, device=q.device)
        for step in range(cp):
            s = (me + step) % cp
            if step == 1:
                comm.barrier(1)
            if s == me:
                q_s, do_s, lse_s, dl_s, acc_s = q, do, lse_pub, delta, dq_tot
            else:
                q_s = comm.view(comm.q, me, (rows, Hq, D), q.dtype, s * comm.q_slot)
                do_s = comm.view(comm.do, me, (rows, Hq, D), q.dtype, s * comm.q_slot)
                lse_s = comm.view(comm.lse, me, (Hq, rows), torch.float32, s * comm.st_slot)
                dl_s = comm.view(comm.delta, me, (Hq, rows), torch.float32, s * comm.st_slot)
                acc_s = torch.zeros(rows, Hq, D, dtype=torch.float32, device=q.device)
            for bi, b in enumerate(_chunk_ids(me, cp)):          # my K/V chunks
                kvn = _valid(b, cs, total)
                for ai, a in enumerate(_chunk_ids(s, cp)):       # the query chunks of rank s
                    qn = _valid(a, cs, total)
                    if a < b or kvn == 0 or qn == 0:
                        continue
                    dk_p = torch.zeros(rows, Hkv, D, dtype=q.dtype, device=q.device)
                    dv_p = torch.zeros_like(dk_p)
                    _C().fa_bwd_ex(q_s, k, v, q_s, do_s, lse_s, dummy, dk_p, dv_p, dl_s, acc_s, _cu(ai * cs, qn, q.device),
                                   _cu(bi * cs, kvn, q.device), (kvn + 127) // 128 + 1, a == b, scale, 1 | 2 | 4, err)
                    dk += dk_p.float()
                    dv += dv_p.float()
            if s != me:
                comm.push(acc_s, comm.dq_acc, me * comm.dq_slot, ranks=[s])   # my share of rank s's dQ, sent once
        if cp > 1:
            comm.barrier(2)
            for s in range(cp):
                if s != me:
                    dq_tot += comm.view(comm.dq_acc, me, (rows, Hq, D), torch.float32, s * comm.dq_slot)
        dq = torch.empty_like(q)
        _C().fa_dq_convert(dq_tot, dq)
        return dq, dk.to(k.dtype), dv.to(v.dtype), None, None, None


def peer_attention(q, k, v, comm: CPComm, total_length: int, scale: Optional[float] = None):
    """Causal attention of one zig-zag-sharded sequence; ``q/k/v`` are this rank's two chunks (bf16, head_dim 128)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _PeerAttention.apply(q, k, v, comm, total_length, float(scale))
