"""Distributed optimizer (ZeRO-1) on flat buffers.

All parameters of a rank are views into ONE contiguous low-precision buffer and
their gradients accumulate into ONE contiguous gradient buffer.  After the
backward passes of a step the gradient buffer is reduce-scattered over the
data-parallel group; every rank runs Adam on its contiguous shard (fp32 state)
and the updated shard is all-gathered back into the parameter buffer - the
behaviour of the reference's always-on distributed optimizer
(relax/backends/megatron/arguments.py:266-289, model.py:282-354,968-1312).

Memory layout choice for 180 GB parts: the fp32 master weight of a bf16
parameter is stored as the bf16 value plus a signed 16-bit remainder
(``fp32_bits == (bf16_bits << 16) + int16``), which reconstructs the fp32
master exactly while saving two bytes per parameter compared with a separate
fp32 copy.  Ten bytes of optimizer state per parameter, spread over dp ranks.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Iterable, Optional

import torch
import torch.distributed as dist

from ..parallel.state import ParallelState


@dataclass
class OptimizerConfig:
    lr: float = 1e-6
    min_lr: float = 0.0
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-8
    clip_grad: float = 1.0
    lr_decay_style: str = "constant"   # constant | linear | cosine
    lr_warmup_iters: int = 0
    lr_decay_iters: Optional[int] = None
    grad_dtype: str = "fp32"           # fp32 | param (accumulate in the parameter dtype)
    split_master: bool = True          # bf16 + int16 remainder instead of an fp32 copy
    fused_dp: bool = True              # reduce-scatter / all-gather inside the optimizer kernels over NVLink peer memory


def lr_at(cfg: OptimizerConfig, it: int) -> float:
    """Learning rate of optimizer step ``it`` (0-based): linear warm-up then the
    chosen decay (relax/backends/megatron/model.py:220-265)."""
    if cfg.lr_warmup_iters > 0 and it < cfg.lr_warmup_iters:
        return cfg.lr * (it + 1) / cfg.lr_warmup_iters
    if cfg.lr_decay_style == "constant" or not cfg.lr_decay_iters:
        return cfg.lr
    t = min(1.0, (it - cfg.lr_warmup_iters) / max(1, cfg.lr_decay_iters - cfg.lr_warmup_iters))
    if cfg.lr_decay_style == "linear":
        c = 1.0 - t
    elif cfg.lr_decay_style == "cosine":
        c = 0.5 * (1.0 + math.cos(math.pi * t))
    else:
        raise ValueError(cfg.lr_decay_style)
    return cfg.min_lr + (cfg.lr - cfg.min_lr) * c


def _split_fp32(x32: torch.Tensor, out_dtype):
    """fp32 -> (low-precision value rounded to nearest, int16 remainder) with
    exact reconstruction for bf16."""
    hi = x32.to(out_dtype)
    hi_bits = hi.view(torch.int16).to(torch.int32) << 16
    rem = x32.view(torch.int32) - hi_bits
    # an exact tie that rounded towards the smaller bit pattern leaves +32768, which
    # does not fit int16: take the other neighbour instead (remainder -32768)
    up = rem == 32768
    hi_bits = torch.where(up, hi_bits + 65536, hi_bits)
    rem = torch.where(up, torch.full_like(rem, -32768), rem)
    hi = (hi_bits >> 16).to(torch.int16).view(out_dtype)
    return hi, rem.to(torch.int16)


def _join_fp32(hi: torch.Tensor, rem: torch.Tensor):
    bits = (hi.view(torch.int16).to(torch.int32) << 16) + rem.to(torch.int32)
    return bits.view(torch.float32)


class DistributedOptimizer:
    ALIGN = 256  # elements; keeps every shard 512-byte aligned

    def __init__(self, model: torch.nn.Module, ps: ParallelState, cfg: OptimizerConfig):
        self.model, self.ps, self.cfg = model, ps, cfg
        params = [p for p in model.parameters() if p.requires_grad]
        self.frozen = [p for p in model.parameters() if not p.requires_grad]
        # replicated-over-TP parameters first: one small all-reduce covers their gradients
        def is_rep(p):
            return getattr(p, "tp_replicated", False)
        self.params = [p for p in params if is_rep(p)] + [p for p in params if not is_rep(p)]
        self.pdtype = self.params[0].dtype
        dev = self.params[0].device
        dp = ps.dp_cp.size
        offs, n = [], 0
        for p in self.params:
            if p.dtype != self.pdtype:
                raise ValueError("all trainable parameters must share one dtype (router weights are kept in "
                                 "fp32 by a separate small optimizer group)")
            offs.append(n)
            n += (p.numel() + 15) // 16 * 16
        self.rep_elems = 0
        for p, o in zip(self.params, offs):
            if is_rep(p):
                self.rep_elems = o + p.numel()
        # parameters that ANOTHER pipeline stage also holds (the last stage's copy of a tied embedding): their
        # gradient is identical on both stages after the tie all-reduce and must enter the global norm once
        self.dup_ranges = [(o, o + p.numel()) for p, o in zip(self.params, offs) if getattr(p, "pp_duplicate", False)]
        chunk = self.ALIGN * dp
        self.total = (n + chunk - 1) // chunk * chunk
        self.shard = self.total // dp
        self.offsets = offs
        gdt = torch.float32 if cfg.grad_dtype == "fp32" else self.pdtype
        self._symm = None
        if (dp > 1 and dev.type == "cuda" and gdt == torch.float32 and self.pdtype == torch.bfloat16
                and getattr(cfg, "fused_dp", True) and os.environ.get("RELAX_B200_FUSED_DP", "1") == "1"):
            self._symm = self._setup_symmetric(dev, dp)
        if self._symm is not None:
            self.param_buf = self._symm["param"].local((self.total,), self.pdtype)
            self.grad_buf = self._symm["grad"].local((self.total,), gdt)
        else:
            self.param_buf = torch.zeros(self.total, dtype=self.pdtype, device=dev)
            self.grad_buf = torch.zeros(self.total, dtype=gdt, device=dev)
        for p, o in zip(self.params, offs):
            v = self.param_buf[o:o + p.numel()].view_as(p)
            v.copy_(p.data)
            p.data = v
            p.main_grad = self.grad_buf[o:o + p.numel()].view_as(p)
            if gdt == self.pdtype:
                p.grad = p.main_grad
            else:
                p.register_post_accumulate_grad_hook(self._make_hook(p))
        r = ps.dp_cp.rank
        self.lo, self.hi = r * self.shard, (r + 1) * self.shard
        my = self.param_buf[self.lo:self.hi]
        self.split_master = cfg.split_master and self.pdtype == torch.bfloat16
        if self.split_master:
            self.master_rem = torch.zeros(self.shard, dtype=torch.int16, device=dev)
            self.master = None
        else:
            self.master = my.float().clone()
        self.exp_avg = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.step_count = 0
        self.grad_shard = None
        self.last_grad_norm = 0.0

    @staticmethod
    def _make_hook(p):
        def hook(param):
            if param.grad is not None:
                param.main_grad.add_(param.grad)
                param.grad = None
        return hook

    # ------------------------------------------------------------------ step pieces
    def zero_grad(self):
        self.grad_buf.zero_()
        if self.grad_buf.dtype == self.pdtype:
            for p in self.params:
                p.grad = p.main_grad

    def _setup_symmetric(self, dev, dp):
        """Parameter and gradient buffers in NVLink-shared memory of the data-parallel group, so the step's
        reduce-scatter and all-gather run inside the optimizer kernels (csrc/dist_optim_sm100.cu).  Returns
        None (NCCL path) when the group does not sit on one node with peer access."""
        import socket

        from ..ops import cuda as C
        from ..parallel.symm_mem import SymmBuffer

        g = self.ps.dp_cp
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        info = [None] * g.size
        dist.all_gather_object(info, (socket.gethostname(), idx), group=g.group)
        ok = len({h for h, _ in info}) == 1 and len({d for _, d in info}) == g.size
        ok = ok and all(C._load().can_access_peer(idx, d) for _, d in info if d != idx)
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=g.group)
        if not int(flag.item()):
            return None
        out = {"param": SymmBuffer(self.total * 2, g, dev), "grad": SymmBuffer(self.total * 4, g, dev),
               "sig": SymmBuffer(1024, g, dev), "state": torch.zeros(16, dtype=torch.int32, device=dev),
               "sumsq": torch.zeros(1, dtype=torch.float32, device=dev),
               "wait_ns": int(os.environ.get("RELAX_B200_PEER_WAIT_MS", "5000")) * 1_000_000}
        torch.cuda.synchronize(dev)
        dist.barrier(group=g.group)
        return out

    def _reduce_grads(self):
        ps = self.ps
        if ps.tp.size > 1 and self.rep_elems > 0:
            dist.all_reduce(self.grad_buf[: self.rep_elems], group=ps.tp.group)
        g = ps.dp_cp
        if self._symm is not None:
            from ..ops import cuda as C

            sy = self._symm
            out = torch.empty(self.shard, dtype=torch.float32, device=self.grad_buf.device)
            sy["sumsq"].zero_()
            C._load().dp_reduce_sumsq(sy["grad"].ptrs, sy["sig"].ptrs, sy["state"], g.rank, self.lo, out, sy["sumsq"],
                                      1.0 / g.size, sy["wait_ns"], C.err_flag(out.device))
            self._fused_sumsq = sy["sumsq"].clone()
            return out
        self._fused_sumsq = None
        if g.size > 1:
            out = torch.empty(self.shard, dtype=self.grad_buf.dtype, device=self.grad_buf.device)
            dist.reduce_scatter_tensor(out, self.grad_buf, op=dist.ReduceOp.SUM, group=g.group)
            out.div_(g.size)
            return out
        return self.grad_buf[self.lo:self.hi]

    def _global_grad_norm(self, gshard: torch.Tensor) -> torch.Tensor:
        ps = self.ps
        # replicated parameters appear on every TP rank: count them once
        lo, hi = self.lo, self.hi
        if getattr(self, "_fused_sumsq", None) is not None:
            tot = self._fused_sumsq[0]      # produced by the fused reduce kernel
            if ps.tp.size > 1 and ps.tp.rank != 0 and self.rep_elems > lo:
                tot = tot - gshard[: max(0, min(hi, self.rep_elems) - lo)].float().pow(2).sum()
        else:
            sq = gshard.float().pow(2)
            tot = sq.sum()
            if ps.tp.size > 1 and ps.tp.rank != 0 and self.rep_elems > lo:
                tot = tot - sq[: max(0, min(hi, self.rep_elems) - lo)].sum()
        for a, b in self.dup_ranges:
            a2, b2 = max(a, lo), min(b, hi)
            if a2 < b2:
                tot = tot - gshard[a2 - lo:b2 - lo].float().pow(2).sum()
        if ps.dp_cp.size > 1:
            dist.all_reduce(tot, group=ps.dp_cp.group)
        if ps.tp.size > 1:
            dist.all_reduce(tot, group=ps.tp.group)
        if ps.pp.size > 1:
            dist.all_reduce(tot, group=ps.pp.group)
        return tot.sqrt()

    def step(self, lr: Optional[float] = None, grad_scale: float = 1.0):
        """Reduce gradients, clip, Adam on my shard, all-gather parameters.
        Returns ``(grad_norm, skipped)``; a non-finite norm skips the update."""
        cfg = self.cfg
        gshard = self._reduce_grads()
        norm = self._global_grad_norm(gshard) * grad_scale
        self.last_grad_norm = float(norm)
        if not math.isfinite(self.last_grad_norm):
            return self.last_grad_norm, True
        clip = 1.0
        if cfg.clip_grad > 0 and self.last_grad_norm > cfg.clip_grad:
            clip = cfg.clip_grad / (self.last_grad_norm + 1e-6)
        self.step_count += 1
        lr = lr if lr is not None else lr_at(cfg, self.step_count - 1)
        g = self.ps.dp_cp
        if self._symm is not None:
            from ..ops import cuda as C

            sy = self._symm   # Adam on my shard + the parameter all-gather, one kernel
            C._load().dp_adam_allgather(sy["param"].ptrs, sy["sig"].ptrs, sy["state"], g.rank, self.lo,
                                        self.master_rem if self.split_master else self.master, gshard, self.exp_avg,
                                        self.exp_avg_sq, self.step_count, lr, cfg.adam_beta1, cfg.adam_beta2, cfg.adam_eps,
                                        cfg.weight_decay, grad_scale * clip, self.split_master, sy["wait_ns"],
                                        C.err_flag(gshard.device))
            return self.last_grad_norm, False
        self._adam_shard(gshard, lr, grad_scale * clip)
        if g.size > 1:
            dist.all_gather_into_tensor(self.param_buf, self.param_buf[self.lo:self.hi].clone(), group=g.group)
        return self.last_grad_norm, False

    def _adam_shard(self, gshard, lr, scale):
        cfg = self.cfg
        pshard = self.param_buf[self.lo:self.hi]
        if gshard.is_cuda:
            from ..ops import cuda as C

            if C.available():
                C.fused_adam(pshard, self.master_rem if self.split_master else self.master, gshard,
                             self.exp_avg, self.exp_avg_sq, self.step_count, lr, cfg.adam_beta1, cfg.adam_beta2,
                             cfg.adam_eps, cfg.weight_decay, scale, self.split_master)
                return
        from ..ops.reference import adam_step

        p32 = _join_fp32(pshard, self.master_rem) if self.split_master else self.master
        p32 = adam_step(p32.clone() if self.split_master else p32, gshard, self.exp_avg, self.exp_avg_sq,
                        self.step_count, lr, cfg.adam_beta1, cfg.adam_beta2, cfg.adam_eps, cfg.weight_decay, scale)
        if self.split_master:
            hi, rem = _split_fp32(p32, self.pdtype)
            pshard.copy_(hi)
            self.master_rem.copy_(rem)
        else:
            pshard.copy_(p32.to(self.pdtype))

    # ------------------------------------------------------------------ state
    def master_shard_fp32(self) -> torch.Tensor:
        return _join_fp32(self.param_buf[self.lo:self.hi], self.master_rem) if self.split_master else self.master

    def state_dict(self) -> dict:
        return {"step": self.step_count, "master": self.master_shard_fp32().cpu(), "exp_avg": self.exp_avg.cpu(),
                "exp_avg_sq": self.exp_avg_sq.cpu(), "shard": (self.lo, self.hi), "total": self.total}

    def load_state_dict(self, sd: dict):
        self.step_count = int(sd["step"])
        m = sd["master"].to(self.exp_avg.device)
        if self.split_master:
            hi, rem = _split_fp32(m, self.pdtype)
            self.param_buf[self.lo:self.hi].copy_(hi)
            self.master_rem.copy_(rem)
        else:
            self.master.copy_(m)
            self.param_buf[self.lo:self.hi].copy_(m.to(self.pdtype))
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        g = self.ps.dp_cp
        if g.size > 1:
            dist.all_gather_into_tensor(self.param_buf, self.param_buf[self.lo:self.hi].clone(), group=g.group)

    def reload_master_from_params(self):
        """After parameters were overwritten in place (checkpoint load, weight
        switch) rebuild the master copy of my shard from them."""
        if self.split_master:
            self.master_rem.zero_()
        else:
            self.master.copy_(self.param_buf[self.lo:self.hi].float())

    def release_grads(self):
        """Drop the gradient buffer (it is zeroed at the start of every step anyway)."""
        if self.grad_buf is None or self._symm is not None:
            return   # symmetric buffers stay mapped on the peers: they are never dropped
        self._grad_meta = (self.grad_buf.shape, self.grad_buf.dtype, self.grad_buf.device)
        self.grad_buf = None
        for p in self.params:
            p.main_grad = None
            p.grad = None

    def _bind_grads(self, buf: torch.Tensor):
        self.grad_buf = buf
        for p, o in zip(self.params, self.offsets):
            p.main_grad = buf[o:o + p.numel()].view_as(p)
            if buf.dtype == self.pdtype:
                p.grad = p.main_grad

    def allocate_grads(self):
        if self.grad_buf is not None:
            return
        shape, dtype, dev = self._grad_meta
        if self._symm is not None:
            # the fused reduce-scatter reads every rank's SYMMETRIC gradient buffer: accumulate there, never in a
            # private tensor
            buf = self._symm["grad"].local(tuple(shape), dtype)
            buf.zero_()
        else:
            buf = torch.zeros(shape, dtype=dtype, device=dev)
        self._bind_grads(buf)

    # ------------------------------------------------------------------ offload (colocate sleep / wake_up)
    def offload_state(self):
        """Move optimizer state to pinned host memory and release the gradient
        buffer (relax/backends/megatron/weight_update/train_offload.py:135-346).  A symmetric gradient buffer
        stays where it is: the peers have it mapped and the fused step reads it by address."""
        self._host = {}
        for name in ("exp_avg", "exp_avg_sq", "master", "master_rem"):
            t = getattr(self, name, None)
            if t is None or not t.is_cuda:
                continue
            h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            h.copy_(t, non_blocking=True)
            self._host[name] = h
        if self.grad_buf is not None and self.grad_buf.is_cuda:
            torch.cuda.current_stream().synchronize()
            for name in self._host:
                setattr(self, name, None)
            if self._symm is None:
                self._grad_meta = (self.grad_buf.shape, self.grad_buf.dtype, self.grad_buf.device)
                self.grad_buf = None
                for p in self.params:
                    p.main_grad = None
                    p.grad = None

    def onload_state(self):
        host = getattr(self, "_host", None)
        if not host:
            return
        dev = self.param_buf.device
        for name, h in host.items():
            setattr(self, name, h.to(dev, non_blocking=True))
        if self.grad_buf is None:
            self.allocate_grads()
        self._host = None

    def close(self):
        """Unmap the peers' symmetric buffers and free this rank's (every rank of the data-parallel group calls
        this, after its last step has completed on the device and before the process groups are destroyed)."""
        sy, self._symm = self._symm, None
        if sy is None:
            return
        for p in self.params:
            p.main_grad = None
            p.grad = None
        self.grad_buf = None
        bufs = [sy[k] for k in ("param", "grad", "sig")]
        for b in bufs:
            b.unmap_peers()
        if dist.is_initialized() and self.ps.dp_cp.size > 1:
            torch.cuda.synchronize()
            dist.barrier(group=self.ps.dp_cp.group)
        for b in bufs:
            b.free_local()
