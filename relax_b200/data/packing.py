"""Packing of variable-length samples into one thd token stream and the index
arithmetic that maps response tokens to logit rows.

Conventions (relax/backends/megatron/data.py:268-605, loss.py:49-191): samples
are concatenated; the stream is padded with a dummy tail sequence to a multiple
of ``pad_multiple`` (``tp * 128`` in the reference); for a sample with total
length ``L`` and response length ``R`` the logits at positions
``[L-R-1, L-1)`` predict the response tokens ``[L-R, L)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch


@dataclass
class PackedBatch:
    tokens: torch.Tensor        # [T] int64
    positions: torch.Tensor     # [T] int64
    cu_seqlens: torch.Tensor    # [B(+1 pad seq)+1] int32
    total_lengths: list
    response_lengths: list
    logit_rows: torch.Tensor    # [sum R] rows of the hidden/logits that predict response tokens
    target_rows: torch.Tensor   # [sum R] rows of ``tokens`` holding the response tokens
    max_seqlen: int
    num_real_tokens: int

    @property
    def targets(self) -> torch.Tensor:
        return self.tokens[self.target_rows]


def pack_samples(token_lists: Sequence, response_lengths: Sequence[int], pad_multiple: int = 1,
                 device="cpu", pad_token: int = 0) -> PackedBatch:
    toks = [torch.as_tensor(t, dtype=torch.int64) for t in token_lists]
    lens = [int(t.numel()) for t in toks]
    total = sum(lens)
    pad = (-total) % pad_multiple
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    pos = [torch.arange(L) for L in lens]
    if pad:
        toks.append(torch.full((pad,), pad_token, dtype=torch.int64))
        pos.append(torch.arange(pad))
        cu.append(cu[-1] + pad)
    tokens = torch.cat(toks) if toks else torch.zeros(0, dtype=torch.int64)
    positions = torch.cat(pos) if pos else torch.zeros(0, dtype=torch.int64)
    lr, tr = [], []
    for i, (L, R) in enumerate(zip(lens, response_lengths)):
        R = int(R)
        s = cu[i]
        lr.append(torch.arange(s + L - R - 1, s + L - 1))
        tr.append(torch.arange(s + L - R, s + L))
    logit_rows = torch.cat(lr) if lr else torch.zeros(0, dtype=torch.int64)
    target_rows = torch.cat(tr) if tr else torch.zeros(0, dtype=torch.int64)
    # one pinned, non-blocking copy for the four index vectors (a blocking copy per tensor would make the host wait for
    # the previous micro-batch's kernels five times per micro-batch)
    from ..algo.ppo_utils import to_device_async

    n_t, n_r = int(tokens.numel()), int(logit_rows.numel())
    flat = to_device_async(torch.cat([tokens, positions, logit_rows, target_rows, torch.tensor(cu, dtype=torch.int64)]), device)
    tokens, positions = flat[:n_t], flat[n_t:2 * n_t]
    logit_rows, target_rows = flat[2 * n_t:2 * n_t + n_r], flat[2 * n_t + n_r:2 * n_t + 2 * n_r]
    cu_dev = flat[2 * n_t + 2 * n_r:].to(torch.int32)
    return PackedBatch(
        tokens=tokens, positions=positions,
        cu_seqlens=cu_dev,
        total_lengths=lens, response_lengths=[int(r) for r in response_lengths],
        logit_rows=logit_rows, target_rows=target_rows,
        max_seqlen=max(lens + ([pad] if pad else [])) if lens else 0, num_real_tokens=total,
    )


def split_by_lengths(x: torch.Tensor, lengths: Sequence[int]) -> list:
    return list(torch.split(x, [int(l) for l in lengths]))
