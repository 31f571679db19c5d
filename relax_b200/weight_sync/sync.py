"""Executors of a weight-sync copy plan.

``WeightSync.update_weights`` follows the reference's protocol (pause ->
flush cache -> move weights -> bump version -> continue;
relax/backends/megatron/weight_update/update_weight_from_tensor.py:178-276,
relax/distributed/checkpoint_service/backends/device_direct.py:598-778), but
moves bytes with block copies from trainer shards directly into the rollout
parameter buffer:

* same process (colocated, equal TP): local strided copies - on CUDA ONE
  launch of the table-driven copy kernel, no staging buffer, no collective;
* different processes: per (src, dst) pair the blocks are packed into one
  message (``torch.distributed`` p2p on CPU/gloo; on CUDA the same kernel
  writes through peer pointers of the symmetric heap).
"""
from __future__ import annotations

import time
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from .plan import BlockCopy, TrainerLayout, build_plan


def _view2d(t: torch.Tensor, batch: int):
    if t.dim() == 3:
        t = t[batch]
    if t.dim() == 1:
        t = t.view(1, -1)
    return t


def apply_block(b: BlockCopy, src: torch.Tensor, dst: torch.Tensor):
    s = _view2d(src, b.src_batch)[b.src_row:b.src_row + b.rows, b.src_col:b.src_col + b.cols]
    d = _view2d(dst, b.dst_batch)[b.dst_row:b.dst_row + b.rows, b.dst_col:b.dst_col + b.cols]
    d.copy_(s)


class WeightSync:
    """Binds one trainer replica to one rollout engine.

    ``trainer_ranks[tp_rank]`` / ``rollout_ranks[tp_rank]`` are GLOBAL ranks.
    Every involved process constructs the object with the same arguments."""

    def __init__(self, cfg: ModelConfig, trainer_layout: TrainerLayout, rollout_tp: int,
                 trainer_ranks: Sequence[int], rollout_ranks: Sequence[int], rollout_ep: int = 1,
                 group=None, post_hook=None, aligned_ep_rank: Optional[int] = None, plan=None):
        self.cfg = cfg
        # ``post_hook(name, tensor) -> tensor`` runs on every rollout tensor after the copy (quantisation round trip)
        self.post_hook = post_hook
        # ``plan``: another list of block copies over the same rank layout (the LoRA factors of adapter-mode sync)
        self.plan = plan if plan is not None else build_plan(cfg, trainer_layout, rollout_tp, rollout_ep)
        # ``trainer_ranks``: list indexed by TP rank (one pipeline stage), or ``{(stage, tp_rank): global rank}``
        if isinstance(trainer_ranks, dict):
            self.trainer_ranks = dict(trainer_ranks)
        else:
            self.trainer_ranks = {(0, i): r for i, r in enumerate(trainer_ranks)}
        self.rollout_ranks = list(rollout_ranks)
        # expert-parallel trainer colocated with an expert-parallel engine on the same ranks (TP 1, equal EP): every
        # rank holds all dense weights and its own experts on both sides, so its whole share is a local copy
        self.aligned_ep_rank = aligned_ep_rank
        self.me = dist.get_rank() if dist.is_initialized() else 0
        self.group = group
        self.last_ms = 0.0
        self._device_table = None

    def _pairs(self):
        pairs: dict = {}
        if self.aligned_ep_rank is not None:
            k = self.aligned_ep_rank
            mine = [b for b in self.plan if (".experts." not in b.src_name) or (b.src_rank == k and b.dst_rank == k)]
            return {(self.me, self.me): mine}
        for b in self.plan:
            s, d = self.trainer_ranks[(b.src_stage, b.src_rank)], self.rollout_ranks[b.dst_rank]
            pairs.setdefault((s, d), []).append(b)
        return pairs

    @torch.no_grad()
    def update_weights(self, trainer_params: Optional[dict], rollout_weights, engine=None, version: Optional[int] = None):
        """``trainer_params``: name -> local shard tensor (None on pure rollout
        ranks); ``rollout_weights``: :class:`RolloutWeights` (None on pure
        trainer ranks)."""
        t0 = time.perf_counter()
        if engine is not None:
            engine.pause_generation()
            if not engine.running:
                engine.flush_cache()
        pairs = self._pairs()
        local = pairs.pop((self.me, self.me), [])
        if local:
            self._local_copy(local, trainer_params, rollout_weights)
        ops_ = []
        recv_bufs = []
        for (s, d), blocks in sorted(pairs.items()):
            n = sum(b.rows * b.cols for b in blocks)
            if s == self.me:
                ref = next(iter(trainer_params.values()))
                buf = torch.empty(n, dtype=ref.dtype, device=ref.device)
                o = 0
                for b in blocks:
                    src = _view2d(trainer_params[b.src_name], b.src_batch)[b.src_row:b.src_row + b.rows, b.src_col:b.src_col + b.cols]
                    buf[o:o + b.rows * b.cols].view(b.rows, b.cols).copy_(src)
                    o += b.rows * b.cols
                ops_.append(dist.P2POp(dist.isend, buf, d, group=self.group))
            elif d == self.me:
                buf = torch.empty(n, dtype=rollout_weights.dtype, device=rollout_weights.device)
                recv_bufs.append((buf, blocks))
                ops_.append(dist.P2POp(dist.irecv, buf, s, group=self.group))
        if ops_:
            for w in dist.batch_isend_irecv(ops_):
                w.wait()
        for buf, blocks in recv_bufs:
            o = 0
            for b in blocks:
                d = _view2d(rollout_weights.p[b.dst_name], b.dst_batch)[b.dst_row:b.dst_row + b.rows, b.dst_col:b.dst_col + b.cols]
                d.copy_(buf[o:o + b.rows * b.cols].view(b.rows, b.cols))
                o += b.rows * b.cols
        if self.post_hook is not None and rollout_weights is not None:
            with torch.no_grad():
                for n, t in rollout_weights.p.items():
                    q = self.post_hook(n, t)
                    if q is not t:
                        t.copy_(q)
        if engine is not None:
            if version is not None:
                engine.update_weight_version(version)
            engine.continue_generation()
        if rollout_weights is not None and rollout_weights.device.type == "cuda":
            torch.cuda.synchronize()
        self.last_ms = (time.perf_counter() - t0) * 1e3
        return self.last_ms

    def _local_copy(self, blocks, trainer_params, rw):
        ref = next(iter(trainer_params.values()))
        if ref.is_cuda:
            from ..ops import cuda as C

            if C.available():
                # the table holds raw addresses: rebuild it whenever either side was re-allocated
                key = (rw.flat.data_ptr(), tuple(trainer_params[b.src_name].data_ptr() for b in blocks[:4]))
                if self._device_table is None or getattr(self, "_table_key", None) != key:
                    self._device_table = C.build_copy_table(blocks, trainer_params, rw)
                    self._table_key = key
                C.run_copy_table(self._device_table)
                return
        for b in blocks:
            apply_block(b, trainer_params[b.src_name], rw.p[b.dst_name])


def oracle_rollout_state(cfg: ModelConfig, full_trainer_state: dict, rollout_tp: int, rollout_rank: int) -> dict:
    """Gather-then-convert oracle: from FULL (unsharded, TP=1) trainer tensors
    build the rollout shard of ``rollout_rank``.  Used by tests to check plans
    bit-exactly."""
    from ..rollout.weights import rollout_param_shapes

    plan = build_plan(cfg, TrainerLayout(1, 1, 1), rollout_tp, 1)
    shapes = rollout_param_shapes(cfg, rollout_tp, 1)
    ref = next(iter(full_trainer_state.values()))
    out = {k: torch.zeros(s, dtype=ref.dtype) for k, s in shapes.items()}
    for b in plan:
        if b.dst_rank == rollout_rank:
            apply_block(b, full_trainer_state[b.src_name], out[b.dst_name])
    return out
