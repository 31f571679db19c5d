"""Symmetric memory over NVLink for the ranks of one process group, and the fused
GEMM + collective operators built on it.

Every rank of the group allocates the same buffers with ``cudaMalloc`` (PyTorch's caching
allocator may use virtual-memory segments, which CUDA IPC cannot export), exchanges the IPC
handles through the group and maps its peers' buffers.  Kernels then store partial results
directly into a peer's workspace and signal through counters in the peer's memory, so the
transfer of one tile overlaps the math of the next and no separate collective is launched.

The reference reaches the same overlap through Megatron's ``--tp-comm-overlap`` (Transformer
Engine userbuffers, relax/utils/arguments.py tp-comm-overlap flags) on the training side and
through the serving engine's custom all-reduce on the rollout side; here both are one family of
sm_100a kernels (csrc/gemm_sm100.cu, epilogue mode 3) that the trainer and the rollout share.

Protocol of one fused call (all ranks issue the same calls in the same order):

* the workspace is double buffered by the parity of a per-rank call counter kept in device
  memory (so CUDA-graph replays advance it without the host);
* a rank's CTAs store fp32 partial tiles into slot ``(parity, rank, k-split)`` of the
  destination's workspace, fence at system scope and add 1 to the destination's arrival
  counter of that parity;
* every CTA then waits - bounded by wall time; on expiry it raises the error flag and leaves -
  until ``tp * grid`` arrivals have been counted locally, and the CTAs reduce the slots row by row
  (plus residual, plus RMSNorm) out of local memory.

A rank can be at most one call ahead of a peer (it cannot complete call ``n+1`` without the
peer's arrivals of call ``n+1``, which the peer issues only after its own call ``n`` has
finished), hence two buffers suffice.
"""
from __future__ import annotations

import os
import socket
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .state import GroupInfo

_SIG_BYTES = 1024


def _C():
    from ..ops import cuda as _cuda

    return _cuda._load()


class SymmBuffer:
    """One symmetric allocation: ``ptrs[r]`` is rank ``r``'s buffer as mapped in this process."""

    def __init__(self, nbytes: int, g: GroupInfo, device: torch.device):
        C = _C()
        self.nbytes, self.g, self.device = int(nbytes), g, device
        self.dev_index = device.index if device.index is not None else torch.cuda.current_device()
        self.local_ptr = C.symm_alloc(self.nbytes, self.dev_index)
        handle = C.ipc_get_handle(self.local_ptr)
        handles: List[Optional[bytes]] = [None] * g.size
        dist.all_gather_object(handles, handle, group=g.group)
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == g.rank:
                self.ptrs.append(self.local_ptr)
            else:
                p = C.ipc_open_handle(h, self.dev_index)
                self._opened.append(p)
                self.ptrs.append(p)

    def local(self, shape, dtype) -> torch.Tensor:
        return _C().tensor_from_ptr(self.local_ptr, list(shape), dtype, self.dev_index)

    def unmap_peers(self):
        C = _C()
        for p in self._opened:
            C.ipc_close(p, self.dev_index)
        self._opened = []

    def free_local(self):
        if self.local_ptr:
            _C().symm_free(self.local_ptr, self.dev_index)
            self.local_ptr = 0

    def close(self, barrier: bool = True):
        """Collective over the group: every rank unmaps its peers' buffers, all ranks meet, then each frees its own.
        Freeing an exported allocation while an importer still has it mapped is undefined in CUDA IPC, so the
        meeting point is not optional when the group is still alive (``barrier=False`` is for callers that close
        several buffers and meet once themselves)."""
        self.unmap_peers()
        if barrier and self.g.size > 1 and dist.is_initialized() and self.local_ptr:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.g.group)
        self.free_local()


def workspace_bytes(tp: int, splits: int, rows_out: int, n: int) -> int:
    """Bytes of the double-buffered fp32 partial-tile workspace of one fused call."""
    return 2 * tp * splits * rows_out * n * 4


class _LocalBuffer:
    """Stand-in for :class:`SymmBuffer` when the group has one rank: a plain device tensor."""

    def __init__(self, nbytes: int, device: torch.device):
        self.nbytes = int(nbytes)
        self.t = torch.zeros(self.nbytes // 4, dtype=torch.int32, device=device)
        self.ptrs = [self.t.data_ptr()]

    def close(self):
        self.t = None
        self.ptrs = []


class SymmComm:
    """Symmetric workspace + arrival counters of one tensor-parallel group and the fused operators
    that use them.  ``workspace_mb`` bounds the largest call (see :func:`workspace_bytes`)."""

    def __init__(self, g: GroupInfo, device: torch.device, workspace_mb: int = 256, wait_ms: Optional[int] = None,
                 gather_mb: Optional[int] = None):
        assert g.size <= 8, "peer tables hold 8 ranks (one NVLink domain)"
        self.g, self.device = g, device
        if g.size == 1:
            # one rank: the same kernels fuse split-K GEMM + reduction + residual + RMSNorm into one launch
            self.ws = _LocalBuffer(workspace_mb << 20, device)
            self.sig = _LocalBuffer(_SIG_BYTES, device)
            self.ag = _LocalBuffer(16, device)
        else:
            self.ws = SymmBuffer(workspace_mb << 20, g, device)
            self.sig = SymmBuffer(_SIG_BYTES, g, device)
            # gathered-activation buffer of the fused all-gather + GEMM ([2][T][K] bf16)
            self.ag = SymmBuffer((gather_mb if gather_mb is not None else workspace_mb // 2) << 20, g, device)
        self.state = torch.zeros(16, dtype=torch.int32, device=device)
        if wait_ms is None:
            wait_ms = int(os.environ.get("RELAX_B200_PEER_WAIT_MS", "5000"))
        self.wait_ns = int(wait_ms) * 1_000_000
        self.calls = 0
        self.timeline = None   # set to an int64 [148, 8] tensor to record per-CTA phase stamps of the next calls
        torch.cuda.synchronize(device)
        if g.size > 1:
            dist.barrier(group=g.group)

    # -- capability switches (callers fall back to the NCCL statement when False)
    def supports(self, op: str) -> bool:
        if self.g.size == 1:
            return op == "gemm_ar_add_rmsnorm"
        return op in ("gemm_ar_add_rmsnorm", "gemm_rs", "ag_gemm")

    def fits_ag(self, shard_rows: int, k: int) -> bool:
        return (shard_rows % 128 == 0 and k % 8 == 0 and
                2 * shard_rows * self.g.size * k * 2 <= self.ag.nbytes)

    def fits(self, rows: int, n: int, splits: int = 8) -> bool:
        """Whether an all-reduce-form call with ``rows`` x ``n`` outputs fits the workspace."""
        if rows > 512:
            return False   # large all-reduces move less data as reduce-scatter + all-gather: leave them to NCCL
        return workspace_bytes(self.g.size, splits, rows, n) <= self.ws.nbytes and n % 32 == 0

    def fits_rs(self, rows: int, n: int) -> bool:
        return workspace_bytes(self.g.size, 1, rows // self.g.size, n) <= self.ws.nbytes and n % 32 == 0

    def _plan(self, M: int, N: int, K: int, reduce_scatter: bool, w_is_kn: bool) -> Tuple[int, int]:
        if reduce_scatter or M > 512:
            # training shapes: large tiles, no split-K
            bn = 256 if N % 256 == 0 else (128 if N % 128 == 0 else 64)
            tm = (M + 127) // 128
            while bn > 64 and tm * (N // bn) < 148:
                bn //= 2
            return 1, bn
        if self.g.size == 1 and os.environ.get("RELAX_B200_LOCAL_PLAN", "splitk") == "splitk":
            # nothing crosses NVLink: take the split-K plan of the plain skinny GEMM (wider N tiles re-read
            # the activation tile from L2 half as often)
            splits, bn = _C().gemm_splitk_plan(M, N, K)
            splits = min(splits, 8)
        else:
            splits, bn = _C().gemm_ar_plan(M, N, K)
        if w_is_kn and bn < 64:
            bn = 64
        return splits, bn

    def _launch(self, x, w, residual, norm_w, eps, reduce_scatter: bool, w_is_kn: bool):
        from ..ops import cuda as _cuda

        M, K = x.shape
        N = w.shape[1] if w_is_kn else w.shape[0]
        tp = self.g.size
        rows_out = M // tp if reduce_scatter else M
        splits, bn = self._plan(M, N, K, reduce_scatter, w_is_kn)
        need = workspace_bytes(tp, splits, rows_out, N)
        if need > self.ws.nbytes:
            raise RuntimeError(f"fused GEMM+collective needs {need >> 20} MiB of symmetric workspace, "
                               f"{self.ws.nbytes >> 20} MiB were set up")
        out_h = torch.empty(rows_out, N, dtype=x.dtype, device=x.device)
        out_x = torch.empty_like(out_h) if norm_w is not None else None
        if x.stride(1) != 1 or (x.stride(0) % 8):
            x = x.contiguous()
        _C().gemm_ar_rmsnorm(x, w, self.ws.ptrs, self.sig.ptrs, self.g.rank, self.state, residual, norm_w, out_h, out_x,
                             float(eps), splits, bn, reduce_scatter, w_is_kn, self.wait_ns, _cuda.err_flag(x.device),
                             self.timeline)
        self.calls += 1
        return out_h, out_x

    def gemm_ar_add_rmsnorm(self, x, w, residual, norm_w, eps):
        """``h = residual + all_reduce(x @ w.T)``; ``y = rmsnorm(h) * norm_w``.  Returns ``(h, y)``
        (``y`` is None without ``norm_w``)."""
        return self._launch(x, w, residual, norm_w, eps, False, False)

    def gemm_rs(self, x, w, w_is_kn: bool = False):
        """``reduce_scatter(x @ w.T)`` over rows: returns this rank's ``[T/tp, N]`` block."""
        return self._launch(x, w, None, None, 0.0, True, w_is_kn)[0]

    def ag_gemm(self, x_shard, w):
        """``all_gather(x_shard, dim=0) @ w.T`` with the gather inside the GEMM kernel: the tiles of this rank's
        own rows are computed while the peers' shards arrive over NVLink.  Returns ``(y, None)``."""
        from ..ops import cuda as _cuda

        Ts, K = x_shard.shape
        N = w.shape[0]
        M = Ts * self.g.size
        bn = 256 if N % 256 == 0 else (128 if N % 128 == 0 else 64)
        while bn > 64 and (M // 128) * (N // bn) < 148:
            bn //= 2
        y = torch.empty(M, N, dtype=x_shard.dtype, device=x_shard.device)
        _C().ag_gemm(x_shard.contiguous(), w, y, self.ag.ptrs, self.sig.ptrs, self.g.rank, self.state, bn, self.wait_ns,
                     _cuda.err_flag(x_shard.device))
        self.calls += 1
        return y, None

    def close(self):
        """Collective over the group (see :meth:`SymmBuffer.close`): unmap everything, meet once, free."""
        bufs = (self.ws, self.sig, self.ag)
        if self.g.size == 1:
            for b in bufs:
                b.close()
            return
        for b in bufs:
            b.unmap_peers()
        if dist.is_initialized() and self.ws.local_ptr:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.g.group)
        for b in bufs:
            b.free_local()


def attach_group(g: GroupInfo, device: torch.device, workspace_mb: int = 256) -> Optional[SymmComm]:
    """Create and register the communicator of ``g`` when every rank of the group sits on one node
    with peer access; returns None (callers keep the NCCL statements) otherwise."""
    from ..ops import fused_comm

    if device.type != "cuda" or os.environ.get("RELAX_B200_FUSED_TP", "1") != "1":
        return None
    if g.size == 1:
        # One rank: the single-launch split-K GEMM + reduce + residual + RMSNorm measured 10-12 us slower per
        # call than the three separate launches inside a CUDA graph (the in-kernel release/wait/reduce tail
        # costs more than two kernel boundaries), so it is opt-in.
        if os.environ.get("RELAX_B200_FUSED_LOCAL", "0") != "1":
            return None
        comm = SymmComm(g, device, min(workspace_mb, 128))
        fused_comm.attach(g, comm)
        return comm
    C = _C()
    dev = device.index if device.index is not None else torch.cuda.current_device()
    # every rank of the group must sit on this host, on a device of its own, with peer access
    info = [None] * g.size
    dist.all_gather_object(info, (socket.gethostname(), dev), group=g.group)
    same_host = len({h for h, _ in info}) == 1 and len({d for _, d in info}) == g.size
    peers_ok = same_host and all(C.can_access_peer(dev, d) for _, d in info if d != dev)
    ok = torch.tensor([1 if peers_ok else 0], device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=g.group)
    if not int(ok.item()):
        return None
    comm = SymmComm(g, device, workspace_mb)
    fused_comm.attach(g, comm)
    return comm
