"""Pipeline parallelism: forward/backward schedules over ``torch.distributed`` p2p.

* :func:`forward_backward_no_pipelining` - gradient accumulation over micro-batches.
* :func:`forward_backward_1f1b` - non-interleaved one-forward-one-backward schedule:
  ``pp - rank - 1`` warm-up forwards, steady 1F1B, cool-down backwards.
* Both accept an *iterator* of micro-batches whose length is not known up front (the
  streaming variants of relax/backends/megatron/streaming_schedules.py:53-457): the first
  stage pulls micro-batches from the data plane as they arrive and tells the later stages
  after each one whether another follows, so the pipeline drains exactly when the stream does.

A stage is described by two callbacks: ``forward_step(mb, input_tensor) -> (output, loss_or_None)``
and the tensors are sent as ``[tokens, hidden]`` activations; shapes travel with a small header
(the reference patches Megatron's shape exchange, docker/patch/latest/megatron.patch:477-560).
Pipeline p2p stays on NCCL (it is latency- not bandwidth-critical and overlaps with compute).
"""
from __future__ import annotations

from typing import Callable, Iterable, Iterator, Optional

import torch
import torch.distributed as dist

from .state import GroupInfo


_PENDING: list = []   # (work, tensor) of sends in flight; sends are asynchronous so that a stage that is
                      # sending activations downstream never blocks a neighbour sending gradients upstream


def _reap(all_: bool = False):
    while _PENDING and (all_ or _PENDING[0][0].is_completed()):
        w, _t = _PENDING.pop(0)
        w.wait()


def _send(t: torch.Tensor, dst: int, group):
    hdr = torch.tensor([t.dim()] + list(t.shape) + [0] * (4 - t.dim()), dtype=torch.int64, device=t.device)
    t = t.contiguous()
    _PENDING.append((dist.isend(hdr, dst, group=group), hdr))
    _PENDING.append((dist.isend(t, dst, group=group), t))
    _reap()


def _recv(src: int, group, device, dtype) -> torch.Tensor:
    hdr = torch.empty(5, dtype=torch.int64, device=device)
    dist.recv(hdr, src, group=group)
    nd = int(hdr[0])
    t = torch.empty([int(x) for x in hdr[1:1 + nd]], dtype=dtype, device=device)
    dist.recv(t, src, group=group)
    return t


def _flag_send(v: int, dst: int, group, device):
    t = torch.tensor([v], dtype=torch.int64, device=device)
    _PENDING.append((dist.isend(t, dst, group=group), t))


def _flag_recv(src: int, group, device) -> int:
    t = torch.empty(1, dtype=torch.int64, device=device)
    dist.recv(t, src, group=group)
    return int(t)


def forward_backward_no_pipelining(microbatches: Iterable, forward_step: Callable, loss_scale: Callable = None):
    """``forward_step(mb, None) -> (output, loss)``; backward after every forward.  Returns the losses."""
    losses = []
    for mb in microbatches:
        _, loss = forward_step(mb, None)
        (loss if loss_scale is None else loss_scale(loss)).backward()
        losses.append(loss.detach())
    return losses


class _Stream:
    """Gives every stage the same view of a micro-batch stream of unknown length: stage 0 owns the
    iterator and forwards a 'more follows' flag down the pipeline with every micro-batch."""

    def __init__(self, it: Optional[Iterator], pp: GroupInfo, device):
        self.it, self.pp, self.device = it, pp, device
        self._next = None
        if pp.rank == 0:
            self._advance()

    def _advance(self):
        try:
            self._next = next(self.it)
        except StopIteration:
            self._next = None

    def pull(self):
        """Stage 0: returns (micro-batch or None).  Later stages: (True/None) from upstream."""
        if self.pp.rank == 0:
            mb = self._next
            if mb is not None:
                self._advance()
            if self.pp.size > 1:
                _flag_send(1 if mb is not None else 0, self.pp.ranks[1], self.pp.group, self.device)
            return mb
        has = _flag_recv(self.pp.ranks[self.pp.rank - 1], self.pp.group, self.device)
        if self.pp.rank + 1 < self.pp.size:
            _flag_send(has, self.pp.ranks[self.pp.rank + 1], self.pp.group, self.device)
        return True if has else None


def forward_backward_1f1b(microbatches: Optional[Iterable], forward_step: Callable, pp: GroupInfo, device, dtype,
                          loss_scale: Callable = None):
    """Non-interleaved 1F1B with a streaming micro-batch source.

    ``forward_step(mb, input_tensor) -> (output_tensor, loss)``: ``mb`` is the micro-batch on stage 0 and
    ``True`` elsewhere (later stages read what they need from ``input_tensor``); the last stage returns the
    loss, the others ``None``.  Returns the list of losses (last stage) or ``[]``."""
    if pp.size == 1:
        return forward_backward_no_pipelining(microbatches, forward_step, loss_scale)
    rank, first, last = pp.rank, pp.rank == 0, pp.rank == pp.size - 1
    prev_r = None if first else pp.ranks[rank - 1]
    next_r = None if last else pp.ranks[rank + 1]
    stream = _Stream(iter(microbatches) if first else None, pp, device)
    in_flight = []   # (input_tensor, output_tensor) awaiting backward
    losses = []

    def fwd(mb):
        x = None
        if not first:
            x = _recv(prev_r, pp.group, device, dtype).requires_grad_()
        out, loss = forward_step(mb, x)
        if not last:
            _send(out.detach(), next_r, pp.group)
            in_flight.append((x, out))
        else:
            losses.append(loss.detach())
            in_flight.append((x, loss if loss_scale is None else loss_scale(loss)))

    def bwd():
        x, out = in_flight.pop(0)
        if last:
            out.backward()
        else:
            g = _recv(next_r, pp.group, device, dtype)
            out.backward(g)
        if not first:
            _send(x.grad, prev_r, pp.group)

    warmup = pp.size - rank - 1
    done = False
    for _ in range(warmup):
        mb = stream.pull()
        if mb is None:
            done = True
            break
        fwd(mb)
    while not done:
        mb = stream.pull()
        if mb is None:
            break
        fwd(mb)
        bwd()
    while in_flight:
        bwd()
    _reap(all_=True)
    return losses
