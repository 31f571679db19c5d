"""Context parallelism: zig-zag sequence layout, loss-side slicing/gathering, dynamic
CP sizing and ring attention.

Layout (relax/backends/megatron/cp_utils.py:39-87): a sequence of length ``L`` is cut
into ``2*cp`` chunks of ``ceil(L / (2*cp))`` tokens; rank ``r`` owns chunk ``r`` and
chunk ``2*cp-1-r`` so causal work is balanced.  Logit rows that predict response
tokens are ``[prompt_len-1, L-1)``; token rows are those +1.

Ring attention here is the unfused statement over ``torch.distributed`` p2p: the K/V
chunks travel around the ring while each rank computes attention of its queries
against the visiting chunks with a running (max, sum) merge.  The fused version reads
the neighbour's K/V tiles from peer memory inside the attention kernel.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .. import ops
from .state import GroupInfo


# ----------------------------------------------------------------------------- layout arithmetic


def chunk_size_of(total_length: int, cp: int, padded_total_length: Optional[int] = None) -> int:
    if padded_total_length is not None:
        if padded_total_length % (2 * cp):
            raise ValueError(f"padded_total_length={padded_total_length} not divisible by 2*cp={2 * cp}")
        return padded_total_length // (2 * cp)
    return (total_length + 2 * cp - 1) // (2 * cp)


def offsets_with_cp(total_length: int, response_length: int, cp: int, rank: int, padded_total_length: Optional[int] = None):
    """Returns ``(chunk_size, chunks, logits, tokens)``, each a pair of ``(start, end)`` for the two
    chunks of ``rank``; empty ranges are ``(0, 0)``.  Offsets count from the start of the prompt."""
    cs = chunk_size_of(total_length, cp, padded_total_length)
    prompt = total_length - response_length
    chunks = ((rank * cs, (rank + 1) * cs), ((2 * cp - rank - 1) * cs, (2 * cp - rank) * cs))
    logits, tokens = [], []
    for a, b in chunks:
        lo, hi = max(a, prompt - 1), min(b, total_length - 1)
        if lo < hi:
            logits.append((lo, hi))
            tokens.append((lo + 1, hi + 1))
        else:
            logits.append((0, 0))
            tokens.append((0, 0))
    return cs, chunks, tuple(logits), tuple(tokens)


def slice_sequence_with_cp(x: torch.Tensor, cp: int, rank: int, pad_value=0) -> torch.Tensor:
    """Local part (two chunks, concatenated) of a full sequence tensor ``[L, ...]``; the tail chunk
    is padded so every rank holds ``2 * chunk`` rows."""
    L = x.shape[0]
    cs = chunk_size_of(L, cp)
    pad = 2 * cp * cs - L
    if pad:
        x = torch.cat([x, x.new_full((pad,) + tuple(x.shape[1:]), pad_value)], 0)
    return torch.cat([x[rank * cs:(rank + 1) * cs], x[(2 * cp - rank - 1) * cs:(2 * cp - rank) * cs]], 0)


def slice_log_prob_with_cp(x: torch.Tensor, total_length: int, response_length: int, cp: int, rank: int,
                           padded_total_length: Optional[int] = None) -> torch.Tensor:
    """Local part of a per-response-token tensor ``[R]`` (log-probs, advantages, masks).  ``padded_total_length``
    is the length the forward sharded the sequence at (a multiple of ``2*cp``); it must be the same value here."""
    if cp == 1:
        return x
    prompt = total_length - response_length
    _, _, logits, _ = offsets_with_cp(total_length, response_length, cp, rank, padded_total_length)
    parts = [x[a - (prompt - 1): b - (prompt - 1)] for a, b in logits if b > a]
    return torch.cat(parts) if parts else x[:0]


def local_num_response_tokens(total_length: int, response_length: int, cp: int, rank: int,
                              padded_total_length: Optional[int] = None) -> int:
    _, _, logits, _ = offsets_with_cp(total_length, response_length, cp, rank, padded_total_length)
    return sum(b - a for a, b in logits)


class _AllReduceDiff(torch.autograd.Function):
    """Differentiable sum all-reduce (backward is the identity on each rank's own contribution
    summed over ranks, i.e. another all-reduce)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def all_gather_with_cp(local: torch.Tensor, total_length: int, response_length: int, g: GroupInfo,
                       padded_total_length: Optional[int] = None) -> torch.Tensor:
    """Rebuild the full ``[R]`` response tensor from CP-local pieces: every rank writes its pieces into a
    zero tensor at their offsets and the tensors are summed (differentiable;
    relax/backends/megatron/cp_utils.py:288-355)."""
    if g.size == 1:
        return local
    prompt = total_length - response_length
    _, _, logits, _ = offsets_with_cp(total_length, response_length, g.size, g.rank, padded_total_length)
    full = local.new_zeros(response_length)
    pieces, o = [], 0
    for a, b in logits:
        n = b - a
        if n > 0:
            pieces.append((a - (prompt - 1), local[o:o + n]))
            o += n
    for start, piece in pieces:
        full = torch.cat([full[:start], piece + full[start:start + piece.numel()], full[start + piece.numel():]])
    return _AllReduceDiff.apply(full, g.group)


def gather_response_with_cp(local: torch.Tensor, total_length: int, response_length: int, g: GroupInfo,
                            padded_total_length: Optional[int] = None) -> torch.Tensor:
    """Full ``[R]`` response tensor on every rank, differentiable ONLY through this rank's own pieces: the value
    is the same everywhere, but a loss computed from it sends gradient to the local tokens alone, so averaging
    parameter gradients over the dp x cp world gives the gradient of the replicated loss exactly once."""
    if g.size == 1:
        return local
    prompt = total_length - response_length
    _, _, logits, _ = offsets_with_cp(total_length, response_length, g.size, g.rank, padded_total_length)
    if local.numel() != sum(b - a for a, b in logits):
        raise ValueError(f"rank {g.rank} holds {local.numel()} response rows, the layout expects "
                         f"{sum(b - a for a, b in logits)} (sequence sharded at a different padded length?)")
    idx, o = [], 0
    for a, b in logits:
        if b > a:
            idx.append(torch.arange(a - (prompt - 1), b - (prompt - 1), device=local.device))
    idx = torch.cat(idx) if idx else torch.zeros(0, dtype=torch.long, device=local.device)
    if idx.numel():
        mine = local.new_zeros(response_length).index_put((idx,), local)
    else:
        # no response row of this sample lives here: stay in the autograd graph all the same, so this rank's
        # backward runs and takes part in the ring exchanges of the ranks that do hold rows
        mine = local.new_zeros(response_length) + local.sum() * 0
    full = mine.detach().clone()
    dist.all_reduce(full, group=g.group)
    return full - mine.detach() + mine


# ----------------------------------------------------------------------------- dynamic CP


def compute_dynamic_cp_size(max_seq_len: int, max_tokens_per_gpu: int, max_cp: int) -> int:
    """Smallest power-of-two CP size (<= max_cp) such that the longest sequence of the micro-batch
    fits the per-GPU token budget (relax/backends/megatron/cp_utils.py:444-455)."""
    cp = 1
    while cp < max_cp and math.ceil(max_seq_len / cp) > max_tokens_per_gpu:
        cp *= 2
    return min(cp, max_cp)


def agree_dynamic_cp_size(local_cp: int, dp_group) -> int:
    """All data-parallel ranks of a micro-batch step must use the same CP size: take the max."""
    if dp_group is None or not dist.is_initialized():
        return local_cp
    t = torch.tensor([local_cp])
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=dp_group)
    return int(t)


def dynamic_cp_subgroup_ranks(cp_ranks: Sequence[int], size: int) -> list:
    """Split the static CP group into consecutive sub-groups of ``size`` ranks."""
    if len(cp_ranks) % size:
        raise ValueError("dynamic CP size must divide the static CP size")
    return [list(cp_ranks[i:i + size]) for i in range(0, len(cp_ranks), size)]


# ----------------------------------------------------------------------------- ring attention (unfused)


def _attn_block(q, k, v, scale, mask):
    """q [Lq,H,D], k/v [Lk,Hkv,D] -> (out fp32 [Lq,H,D] un-normalised, m [Lq,H], l [Lq,H])."""
    Hq, Hkv = q.shape[1], k.shape[1]
    g = Hq // Hkv
    kk = k.float().repeat_interleave(g, 1)
    vv = v.float().repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->qhk", q.float(), kk) * scale
    if mask is not None:
        s = s.masked_fill(~mask[:, None, :], float("-inf"))
    m = s.amax(-1)
    m_safe = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    p = torch.exp(s - m_safe[..., None])
    l = p.sum(-1)
    o = torch.einsum("qhk,khd->qhd", p, vv)
    return o, m, l


class _RingAttention(torch.autograd.Function):
    """Single-sequence zig-zag causal ring attention.  q/k/v are the LOCAL rows (two chunks)."""

    @staticmethod
    def forward(ctx, q, k, v, g: GroupInfo, total_length: int, scale: float):
        cp, r = g.size, g.rank
        cs = q.shape[0] // 2
        qpos = torch.cat([torch.arange(r * cs, (r + 1) * cs), torch.arange((2 * cp - r - 1) * cs, (2 * cp - r) * cs)]).to(q.device)
        o = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        m = torch.full(q.shape[:2], float("-inf"), device=q.device)
        l = torch.zeros(q.shape[:2], device=q.device)
        kv = torch.stack([k, v]).contiguous()
        for step in range(cp):
            src = (r - step) % cp
            kpos = torch.cat([torch.arange(src * cs, (src + 1) * cs), torch.arange((2 * cp - src - 1) * cs, (2 * cp - src) * cs)]).to(q.device)
            mask = (kpos[None, :] <= qpos[:, None]) & (kpos[None, :] < total_length)
            if step + 1 < cp:
                nxt = torch.empty_like(kv)
                ops_ = [dist.P2POp(dist.isend, kv, g.ranks[(r + 1) % cp], group=g.group),
                        dist.P2POp(dist.irecv, nxt, g.ranks[(r - 1) % cp], group=g.group)]
                reqs = dist.batch_isend_irecv(ops_)
            ob, mb, lb = _attn_block(q, kv[0], kv[1], scale, mask)
            m_new = torch.maximum(m, mb)
            m_new_safe = torch.where(torch.isfinite(m_new), m_new, torch.zeros_like(m_new))
            a = torch.where(torch.isfinite(m), torch.exp(m - m_new_safe), torch.zeros_like(m))
            b = torch.where(torch.isfinite(mb), torch.exp(mb - m_new_safe), torch.zeros_like(mb))
            o = o * a[..., None] + ob * b[..., None]
            l = l * a + lb * b
            m = m_new
            if step + 1 < cp:
                for w in reqs:
                    w.wait()
                kv = nxt
        out = o / l.clamp_min(1e-30)[..., None]
        lse = torch.where(torch.isfinite(m), m, torch.zeros_like(m)) + torch.log(l.clamp_min(1e-30))
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.g, ctx.total_length, ctx.scale, ctx.cs = g, total_length, scale, cs
        return out.to(q.dtype)

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        g, cp, r, cs, scale = ctx.g, ctx.g.size, ctx.g.rank, ctx.cs, ctx.scale
        Hq, Hkv = q.shape[1], k.shape[1]
        grp = Hq // Hkv
        qpos = torch.cat([torch.arange(r * cs, (r + 1) * cs), torch.arange((2 * cp - r - 1) * cs, (2 * cp - r) * cs)]).to(q.device)
        do = do.float()
        delta = (out * do).sum(-1)                      # [Lq, H]
        dq = torch.zeros_like(q, dtype=torch.float32)
        kv = torch.stack([k, v]).contiguous()
        dkv = torch.zeros(kv.shape, dtype=torch.float32, device=q.device)   # travels with kv
        for step in range(cp):
            src = (r - step) % cp
            kpos = torch.cat([torch.arange(src * cs, (src + 1) * cs), torch.arange((2 * cp - src - 1) * cs, (2 * cp - src) * cs)]).to(q.device)
            mask = (kpos[None, :] <= qpos[:, None]) & (kpos[None, :] < ctx.total_length)
            kk = kv[0].float().repeat_interleave(grp, 1)
            vv = kv[1].float().repeat_interleave(grp, 1)
            s = torch.einsum("qhd,khd->qhk", q.float(), kk) * scale
            p = torch.exp(s - lse[..., None]).masked_fill(~mask[:, None, :], 0.0)
            dv_e = torch.einsum("qhk,qhd->khd", p, do)
            dp = torch.einsum("qhd,khd->qhk", do, vv)
            ds = p * (dp - delta[..., None]) * scale
            dq += torch.einsum("qhk,khd->qhd", ds, kk)
            dk_e = torch.einsum("qhk,qhd->khd", ds, q.float())
            dkv[0] += dk_e.view(-1, Hkv, grp, k.shape[-1]).sum(2)
            dkv[1] += dv_e.view(-1, Hkv, grp, k.shape[-1]).sum(2)
            # pass kv and its gradient accumulator to the next rank; after cp steps both are home again
            nkv, ndkv = torch.empty_like(kv), torch.empty_like(dkv)
            reqs = dist.batch_isend_irecv([
                dist.P2POp(dist.isend, kv, g.ranks[(r + 1) % cp], group=g.group),
                dist.P2POp(dist.irecv, nkv, g.ranks[(r - 1) % cp], group=g.group),
                dist.P2POp(dist.isend, dkv, g.ranks[(r + 1) % cp], group=g.group),
                dist.P2POp(dist.irecv, ndkv, g.ranks[(r - 1) % cp], group=g.group)])
            for w in reqs:
                w.wait()
            kv, dkv = nkv, ndkv
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None


def ring_attention(q, k, v, g: GroupInfo, total_length: int, scale: Optional[float] = None):
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if g.size == 1:
        cu = torch.tensor([0, q.shape[0]], dtype=torch.int32, device=q.device)
        return ops.attention_varlen(q, k, v, cu, causal=True, scale=scale)
    return _RingAttention.apply(q, k, v, g, total_length, scale)


def allgather_attention(q, k, v, g: GroupInfo, total_length: int, scale: Optional[float] = None):
    """The all-gather variant of context parallelism (``--allgather-cp``): K and V of the whole sequence are gathered
    on every rank (backward: their gradients are summed and each rank keeps its rows), and each of the rank's two
    zig-zag query chunks attends to the key prefix that ends with it - two calls of the ordinary causal attention
    operator with a query block shorter than its keys, no ring, no partial-result merging.  Costs ``O(L)`` K/V
    memory per rank instead of ``O(L / cp)``; fewer, larger attention calls."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if g.size == 1:
        cu = torch.tensor([0, q.shape[0]], dtype=torch.int32, device=q.device)
        return ops.attention_varlen(q, k, v, cu, causal=True, scale=scale)
    cp, r = g.size, g.rank
    cs = q.shape[0] // 2
    kf = _GatherZigzag.apply(k.contiguous(), g)
    vf = _GatherZigzag.apply(v.contiguous(), g)
    outs = []
    for ai, a in enumerate((r, 2 * cp - 1 - r)):
        qn = max(0, min(cs, total_length - a * cs))        # real rows of this chunk
        qa = q[ai * cs:(ai + 1) * cs]
        if qn == 0:
            outs.append(qa * 0)
            continue
        klen = a * cs + qn
        cu_q = torch.tensor([0, qn], dtype=torch.int32, device=q.device)
        cu_k = torch.tensor([0, klen], dtype=torch.int32, device=q.device)
        o = ops.attention_varlen(qa[:qn].contiguous(), kf[:klen], vf[:klen], cu_q, causal=True, scale=scale,
                                 cu_seqlens_k=cu_k, max_seqlen=klen)
        if qn < cs:
            o = torch.cat([o, qa[qn:] * 0])
        outs.append(o)
    return torch.cat(outs)


# --------------------------------------------------------------------------- whole-sequence ops under CP
class _GatherZigzag(torch.autograd.Function):
    """Local zig-zag shard ``[2 * cs, ...]`` -> the full sequence ``[2 * cp * cs, ...]`` in token order on every rank.
    Backward keeps this rank's rows of the summed gradient (an all-reduce followed by the slice, i.e. a
    reduce-scatter in zig-zag order)."""

    @staticmethod
    def forward(ctx, x, g: GroupInfo):
        ctx.g = g
        cp, cs = g.size, x.shape[0] // 2
        parts = [torch.empty_like(x) for _ in range(cp)]
        dist.all_gather(parts, x.contiguous(), group=g.group)
        full = x.new_empty((2 * cp * cs,) + tuple(x.shape[1:]))
        for r, p in enumerate(parts):
            full[r * cs:(r + 1) * cs] = p[:cs]
            full[(2 * cp - 1 - r) * cs:(2 * cp - r) * cs] = p[cs:]
        return full

    @staticmethod
    def backward(ctx, dy):
        g = ctx.g
        cp, r = g.size, g.rank
        cs = dy.shape[0] // (2 * cp)
        dy = dy.contiguous()
        dist.all_reduce(dy, group=g.group)
        return torch.cat([dy[r * cs:(r + 1) * cs], dy[(2 * cp - 1 - r) * cs:(2 * cp - r) * cs]]), None


def zigzag_rows(cp: int, rank: int, cs: int, device=None) -> torch.Tensor:
    return torch.cat([torch.arange(rank * cs, (rank + 1) * cs, device=device),
                      torch.arange((2 * cp - 1 - rank) * cs, (2 * cp - rank) * cs, device=device)])


def run_on_full_sequence(fn, x_local: torch.Tensor, g: GroupInfo) -> torch.Tensor:
    """Apply a token mixer that needs the whole sequence in order (a recurrence such as the gated delta rule, a
    causal convolution) to a context-parallel shard: gather the sequence, run ``fn`` on it on every rank, keep this
    rank's zig-zag rows (relax/backends/megatron/cp_utils.py GDN helpers :658-774: all-gather forward,
    reduce-scatter backward).  Each rank divides its output gradient contribution by ``cp`` implicitly: only the
    local rows of ``fn``'s output are used, so the summed input gradient is exact."""
    if g.size == 1:
        return fn(x_local)
    full = _GatherZigzag.apply(x_local, g)
    y = fn(full)
    return y.index_select(0, zigzag_rows(g.size, g.rank, x_local.shape[0] // 2, y.device))
