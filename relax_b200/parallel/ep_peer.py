"""Expert-parallel token exchange over NVLink symmetric memory.

The MoE dispatch and combine are variable-size all-to-alls of token rows.  Here a rank writes its rows for
expert-owner ``d`` straight into ``d``'s receive buffer with peer stores (one copy kernel per destination, offsets
computed from the count matrix every rank holds after a small count exchange done the same way), and a barrier
kernel on the signal pads replaces the collective's completion.  The receive buffer is ordered by source rank,
as ``all_to_all_single`` orders it, so :class:`_PeerAllToAll` is a drop-in for the NCCL statement in
``relax_b200/models/moe.py`` (the reference: Megatron's ``alltoall`` token dispatcher, or DeepEP's NVSHMEM
kernels with ``--moe-flex-dispatcher-backend deepep``, scripts/training/text/run-qwen3-30B-A3B-8xgpu.sh:91-93).
The backward of an exchange is the exchange with the split lists swapped.
"""
from __future__ import annotations

import os
from typing import List, Sequence

import torch

from .state import GroupInfo
from .symm_mem import SymmBuffer


def _C():
    from ..ops import cuda as C

    return C._load()


class EPComm:
    def __init__(self, g: GroupInfo, device, capacity_rows: int, hidden: int, elem_size: int = 2, max_experts: int = 512):
        assert g.size <= 8
        self.g, self.device = g, torch.device(device)
        self.dev = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.cap, self.hidden, self.esz = capacity_rows, hidden, elem_size
        self.slot = capacity_rows * hidden * elem_size
        self.recv = SymmBuffer(2 * self.slot, g, self.device)               # double buffered by call parity
        self.cnt_slot = (max_experts * 8 + 15) // 16 * 16
        self.counts = SymmBuffer(2 * g.size * self.cnt_slot, g, self.device)  # [parity][src][experts] int64
        self.sig = SymmBuffer(1024, g, self.device)
        self.state = torch.zeros(16, dtype=torch.int32, device=self.device)
        self.wait_ns = int(os.environ.get("RELAX_B200_PEER_WAIT_MS", "5000")) * 1_000_000
        self.calls = self.count_calls = 0
        torch.cuda.synchronize(self.device)
        import torch.distributed as dist

        dist.barrier(group=g.group)

    def _barrier(self, slot: int):
        from ..ops import cuda as C

        _C().peer_barrier(self.sig.ptrs, self.state, self.g.rank, slot, slot, self.wait_ns, C.err_flag(self.device))

    def exchange_counts(self, counts: torch.Tensor) -> torch.Tensor:
        """``counts [E]`` (int64, tokens this rank routes to every global expert) -> ``[ep, E]`` of all ranks."""
        n, me = self.g.size, self.g.rank
        E = counts.numel()
        if E * 8 > self.cnt_slot:
            raise ValueError("more experts than the count table holds")
        parity = self.count_calls & 1
        self.count_calls += 1
        pad = torch.zeros(self.cnt_slot // 8, dtype=torch.int64, device=self.device)
        pad[:E] = counts
        off = (parity * n + me) * self.cnt_slot
        _C().peer_push(pad, self.counts.ptrs, off)          # every rank, including this one
        self._barrier(0)
        tab = _C().tensor_from_ptr(self.counts.ptrs[me] + parity * n * self.cnt_slot, [n, self.cnt_slot // 8], torch.int64, self.dev)
        return tab[:, :E].clone()

    def all_to_all(self, x: torch.Tensor, send_matrix: Sequence[Sequence[int]]) -> torch.Tensor:
        """``x`` rows grouped by destination rank; ``send_matrix[s][d]`` = rows rank ``s`` sends to rank ``d``
        (the same matrix on every rank).  Returns the rows this rank receives, ordered by source rank."""
        n, me = self.g.size, self.g.rank
        x = x.contiguous()
        row_bytes = x.shape[1] * x.element_size()
        recv_rows = sum(send_matrix[s][me] for s in range(n))
        if max(sum(send_matrix[s][d] for s in range(n)) for d in range(n)) * row_bytes > self.slot:
            raise RuntimeError("MoE exchange exceeds the receive buffer; raise capacity_rows")
        parity = self.calls & 1
        self.calls += 1
        start = 0
        for d in range(n):
            cnt = send_matrix[me][d]
            if cnt:
                off_rows = sum(send_matrix[s][d] for s in range(me))
                seg = x[start:start + cnt]
                if (seg.data_ptr() % 16) or (off_rows * row_bytes % 16) or (cnt * row_bytes % 16):
                    raise ValueError("rows must be multiples of 16 bytes")
                _C().peer_push(seg, [self.recv.ptrs[d]], parity * self.slot + off_rows * row_bytes)
            start += cnt
        self._barrier(1)
        out = _C().tensor_from_ptr(self.recv.ptrs[me] + parity * self.slot, [recv_rows, x.shape[1]], x.dtype, self.dev)
        return out.clone()      # the buffer is reused two calls later; autograd may keep this tensor longer

    def close(self):
        for b in (self.recv, self.counts, self.sig):
            b.close()


class _PeerAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send_matrix, comm: EPComm):
        ctx.comm, ctx.matrix = comm, send_matrix
        return comm.all_to_all(x, send_matrix)

    @staticmethod
    def backward(ctx, dy):
        m = ctx.matrix
        n = len(m)
        transposed = [[m[d][s] for d in range(n)] for s in range(n)]
        return ctx.comm.all_to_all(dy.contiguous(), transposed), None, None


def peer_all_to_all(x: torch.Tensor, send_matrix: List[List[int]], comm: EPComm) -> torch.Tensor:
    return _PeerAllToAll.apply(x, send_matrix, comm)
