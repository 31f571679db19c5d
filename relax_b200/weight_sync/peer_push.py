"""Trainer -> rollout weight push into ANOTHER process's parameter buffer.

In fully-asynchronous and hybrid modes trainer ranks and rollout ranks are different processes on different GPUs.
The reference moves every tensor with one NCCL broadcast from the trainer to all engines
(relax/backends/megatron/weight_update/update_weight_from_distributed.py:351-376,
relax/distributed/checkpoint_service/backends/device_direct.py:598-778: gather the full tensor, convert names
and layout, broadcast, let every engine cut out its shard).  Here each trainer rank maps the parameter buffers of
the rollout ranks it feeds into its own address space and ONE launch of the table-driven copy kernel
(``rb_copy_table``) reads its shards and stores them - resharded TP->TP and converted from the Megatron layout to
the serving layout by the block-copy plan - straight into those buffers over NVLink.  No staging buffer, no
collective, and only the bytes a destination needs cross the link.

How the mapping is made: the rollout buffer is a CUDA virtual-memory allocation created exportable as a POSIX
file descriptor (csrc/vmm.cpp); the owner hands the descriptor to the trainer process over a Unix socket
(:mod:`relax_b200.utils.fd_channel`), which imports and maps it (``cuMemImportFromShareableHandle``).  On the CPU
(tests) the buffer lives in a shared-memory file that the trainer process maps - same code path, plain copies.

:class:`BroadcastPusher` is the baseline arm: the same plan executed as one ``torch.distributed`` broadcast of
each source rank's packed blocks plus local unpacking on the receivers.
"""
from __future__ import annotations

import math
import os
import time
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..rollout.weights import rollout_layout
from ..utils.fd_channel import FdServer, fetch_fds, socket_path
from .plan import BlockCopy, TrainerLayout, build_plan
from .sync import _view2d, apply_block


class SharedWeightRegion:
    """Owner side (a rollout rank): lets other processes of the node map this rank's flat weight buffer."""

    def __init__(self, weights, tag: str, rank: int):
        self.weights = weights
        self.path = socket_path(tag, rank)
        if weights.device.type == "cuda":
            if not weights.memory_saver or weights._buf is None:
                raise ValueError("the weight buffer must be a pausable (virtual-memory) allocation to be exported")
            buf = weights._buf
            C = buf._C

            def provide():
                return {"nbytes": int(C.vmm_size(buf._ptr)), "numel": weights.numel}, [int(C.vmm_export_fd(buf._ptr))]
        else:
            if weights.shared_path is None:
                raise ValueError("on the CPU the weight buffer must be backed by a shared-memory file (shared_path)")

            def provide():
                return {"shm": weights.shared_path, "numel": weights.numel}, []
        self.server = FdServer(self.path, provide)

    def close(self):
        self.server.close()


class _PtrView:
    """Address arithmetic over a row-major tensor that lives in ANOTHER GPU's memory.  Deliberately not a
    ``torch.Tensor``: nothing but the copy kernel's address table may touch peer memory (a library kernel handed a
    peer pointer could issue loads that are not safe across GPUs), so the view only answers the questions the table
    builder asks."""

    def __init__(self, ptr: int, shape, itemsize: int):
        self.ptr, self.shape, self.itemsize = int(ptr), tuple(int(x) for x in shape), int(itemsize)

    def dim(self) -> int:
        return len(self.shape)

    def data_ptr(self) -> int:
        return self.ptr

    def stride(self, d: int) -> int:
        return int(math.prod(self.shape[d + 1:]))

    def __getitem__(self, i: int) -> "_PtrView":
        return _PtrView(self.ptr + int(i) * self.stride(0) * self.itemsize, self.shape[1:], self.itemsize)

    def view(self, *shape) -> "_PtrView":
        n = math.prod(self.shape)
        shape = tuple(n // max(1, -math.prod(shape)) if x == -1 else x for x in shape)
        return _PtrView(self.ptr, shape, self.itemsize)


class PeerRegion:
    """Importer side (a trainer rank): another rank's flat weight buffer mapped here, with per-parameter views."""

    def __init__(self, cfg: ModelConfig, rollout_tp: int, tag: str, owner_rank: int, device, dtype, rollout_ep: int = 1,
                 timeout: float = 120.0, mtp: bool = False):
        self.device, self.dtype = torch.device(device), dtype
        shapes, offsets, numel = rollout_layout(cfg, rollout_tp, rollout_ep, mtp)
        payload, fds = fetch_fds(socket_path(tag, owner_rank), timeout=timeout)
        if int(payload["numel"]) != numel:
            raise RuntimeError(f"rollout rank {owner_rank} holds {payload['numel']} elements, the layout says {numel}")
        self._ptr, self._C = 0, None
        if "shm" in payload:
            self.flat = torch.from_file(payload["shm"], shared=True, size=numel, dtype=dtype)
        else:
            from ..ops import cuda as C

            self._C = C._load()
            idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
            try:
                self._ptr = self._C.vmm_import_fd(int(fds[0]), int(payload["nbytes"]), idx)
            finally:
                for fd in fds:
                    os.close(fd)
            self.flat = None
        if self.flat is not None:
            self.p = {k: self.flat[o:o + math.prod(shapes[k])].view(shapes[k]) for k, o in offsets.items()}
        else:
            es = torch.empty(0, dtype=dtype).element_size()
            self.p = {k: _PtrView(self._ptr + o * es, shapes[k], es) for k, o in offsets.items()}
        if cfg.tie_word_embeddings:
            self.p["lm_head"] = self.p["embed"]

    def close(self):
        self.p, self.flat = {}, None
        if self._ptr and self._C is not None:
            self._C.vmm_unimport(self._ptr)
            self._ptr = 0


class PeerWeightPusher:
    """One trainer rank's part of a weight push: every plan block whose source is this rank, for every engine it
    feeds.  ``engines`` is a list of global-rank lists (one per engine, ordered by the engine's TP rank)."""

    def __init__(self, cfg: ModelConfig, trainer_layout: TrainerLayout, rollout_tp: int, my_src_rank: int,
                 engines: Sequence[Sequence[int]], tag: str, device, dtype, mtp: bool = False):
        # ``mtp``: the engines also hold the first multi-token-prediction block (they speculate with it)
        self.cfg, self.device = cfg, torch.device(device)
        plan = build_plan(cfg, trainer_layout, rollout_tp, 1, mtp=mtp)
        self.regions: dict = {}
        self.work: list = []      # (region, blocks)
        for eng in engines:
            for j, grank in enumerate(eng):
                blocks = [b for b in plan if b.src_rank == my_src_rank and b.dst_rank == j]
                if not blocks:
                    continue
                if grank not in self.regions:
                    self.regions[grank] = PeerRegion(cfg, rollout_tp, tag, grank, device, dtype, mtp=mtp)
                self.work.append((self.regions[grank], blocks))
        self.bytes_per_push = sum(b.rows * b.cols for _, bl in self.work for b in bl) * torch.empty(0, dtype=dtype).element_size()
        self._table, self._key = None, None
        self.last_ms = 0.0

    @torch.no_grad()
    def push(self, trainer_params: dict) -> float:
        """Copies this rank's blocks into every destination buffer; returns the milliseconds it took on the device
        (CUDA events) or on the host (CPU)."""
        if not self.work:
            return 0.0
        if self.device.type == "cuda":
            from ..ops import cuda as C

            key = tuple(trainer_params[bl[0].src_name].data_ptr() for _, bl in self.work)
            if self._table is None or self._key != key:
                entries = []
                for region, blocks in self.work:
                    entries += C.copy_entries(blocks, trainer_params, region.p)
                es = next(iter(trainer_params.values())).element_size()
                self._table = C.build_copy_table_raw(entries, self.device, es)
                self._table.keepalive = (trainer_params, self.regions)
                self._key = key
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            C.run_copy_table(self._table)
            e1.record()
            e1.synchronize()
            self.last_ms = e0.elapsed_time(e1)
        else:
            t0 = time.perf_counter()
            for region, blocks in self.work:
                for b in blocks:
                    apply_block(b, trainer_params[b.src_name], region.p[b.dst_name])
            self.last_ms = (time.perf_counter() - t0) * 1e3
        return self.last_ms

    def close(self):
        self._table = None
        for r in self.regions.values():
            r.close()
        self.regions = {}


class BroadcastPusher:
    """Baseline: the same plan moved by collectives.  For every source trainer rank one broadcast of its packed
    blocks (the union over destinations) inside ``group`` (source + all destination ranks); receivers unpack the
    blocks that are theirs.  Every member of the group calls :meth:`sync` (``trainer_params`` None on receivers,
    ``rollout_weights`` None on sources)."""

    def __init__(self, cfg: ModelConfig, trainer_layout: TrainerLayout, rollout_tp: int, src_global_ranks: Sequence[int],
                 engines: Sequence[Sequence[int]], group, device, dtype, src_index: Optional[int] = None, mtp: bool = False):
        # ``src_index``: this object moves the blocks of ONE source rank (its group holds that rank and the
        # destinations); None: all sources through one group that contains them all
        self.src_index = src_index
        self.plan = build_plan(cfg, trainer_layout, rollout_tp, 1, mtp=mtp)
        self.src, self.engines, self.group = list(src_global_ranks), [list(e) for e in engines], group
        self.device, self.dtype = torch.device(device), dtype
        self.me = dist.get_rank() if dist.is_initialized() else 0
        self.last_ms = 0.0

    @torch.no_grad()
    def sync(self, trainer_params: Optional[dict], rollout_weights) -> float:
        t0 = time.perf_counter()
        my_tp = next((j for e in self.engines for j, g in enumerate(e) if g == self.me), None)
        for s, src_global in enumerate(self.src):
            if self.src_index is not None and s != self.src_index:
                continue
            blocks = [b for b in self.plan if b.src_rank == s]
            # identical (src tensor, rows, cols) regions are sent once even when several destinations take them
            uniq, order = {}, []
            for b in blocks:
                k = (b.src_name, b.src_batch, b.src_row, b.src_col, b.rows, b.cols)
                if k not in uniq:
                    uniq[k] = sum(x[4] * x[5] for x in order)
                    order.append(k)
            n = sum(k[4] * k[5] for k in order)
            buf = torch.empty(n, dtype=self.dtype, device=self.device)
            if self.me == src_global:
                for k in order:
                    name, batch, r0, c0, rows, cols = k
                    src = _view2d(trainer_params[name], batch)[r0:r0 + rows, c0:c0 + cols]
                    buf[uniq[k]:uniq[k] + rows * cols].view(rows, cols).copy_(src)
            dist.broadcast(buf, src=src_global, group=self.group)
            if my_tp is not None and rollout_weights is not None:
                for b in blocks:
                    if b.dst_rank != my_tp:
                        continue
                    o = uniq[(b.src_name, b.src_batch, b.src_row, b.src_col, b.rows, b.cols)]
                    d = _view2d(rollout_weights.p[b.dst_name], b.dst_batch)[b.dst_row:b.dst_row + b.rows, b.dst_col:b.dst_col + b.cols]
                    d.copy_(buf[o:o + b.rows * b.cols].view(b.rows, b.cols))
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        self.last_ms = (time.perf_counter() - t0) * 1e3
        return self.last_ms
