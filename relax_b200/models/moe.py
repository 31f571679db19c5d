"""Mixture-of-experts MLP with expert parallelism.

Softmax router in fp32, top-k, token permutation, all-to-all dispatch to the
ranks that own the experts, grouped SwiGLU expert GEMMs, all-to-all combine and
weighted un-permutation - the pipeline the reference configures through
Megatron (scripts/models/qwen3-30B-A3B.sh:40-50: alltoall dispatcher, grouped
GEMM, permute fusion).  This file is the unfused statement over
``torch.distributed``; on CUDA the dispatch+permute+grouped-GEMM and
GEMM+unpermute+combine pairs are fused kernels (:mod:`relax_b200.ops.fused_comm`).

Routing replay (relax/utils/training/routing_replay.py:17-106): when a
:class:`RoutingReplay` is active the top-k indices recorded by an earlier
forward (rollout or old-policy) replace the router's own choice, while the
gate weights are still computed from the current router logits.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..parallel.state import ParallelState


class RoutingReplay:
    """Process-wide record/replay switch for MoE top-k decisions."""

    mode: Optional[str] = None  # None | "record" | "replay"
    store: dict = {}
    cursor: dict = {}
    # per-sample form: when a layout (sample ids and token counts of the packed micro-batch) is set, decisions are
    # stored per (layer, sample) and re-assembled for whatever micro-batch the sample lands in at replay time, so
    # the recording forward and the training forward may pack their micro-batches differently
    layout: Optional[tuple] = None
    per_sample: dict = {}

    @classmethod
    def set_layout(cls, sample_ids, lengths):
        cls.layout = (list(sample_ids), [int(x) for x in lengths]) if sample_ids is not None else None

    @classmethod
    def begin_record(cls):
        cls.mode, cls.store, cls.per_sample = "record", {}, {}

    @classmethod
    def begin_replay(cls, store: Optional[dict] = None):
        cls.mode = "replay"
        if store is not None:
            cls.store = store
        cls.cursor = {k: 0 for k in cls.store}

    @classmethod
    def end(cls):
        cls.mode, cls.layout = None, None

    @classmethod
    def route(cls, layer_idx: int, idx: torch.Tensor) -> torch.Tensor:
        if cls.mode is not None and cls.layout is not None:
            ids, lens = cls.layout
            if sum(lens) > idx.shape[0]:
                raise ValueError("per-sample routing replay needs the whole packed micro-batch on this rank (tp = 1)")
            if cls.mode == "record":
                o = 0
                for sid, n in zip(ids, lens):
                    cls.per_sample[(layer_idx, sid)] = idx[o:o + n].detach().clone()
                    o += n
                return idx
            parts, o = [], 0
            for sid, n in zip(ids, lens):
                rec = cls.per_sample.get((layer_idx, sid))
                if rec is not None and rec.shape[0] == n - 1:
                    # recorded by the rollout engine: it never feeds a sample's last token, whose row keeps the
                    # router's own choice (no loss is taken at that position)
                    rec = torch.cat([rec.to(idx.device), idx[o + n - 1:o + n]])
                if rec is None or rec.shape[0] != n:
                    raise ValueError(f"no recorded routing for sample {sid} at layer {layer_idx}")
                parts.append(rec.to(idx.device))
                o += n
            tail = idx[sum(lens):]                       # padding rows keep the router's own choice
            return torch.cat(parts + [tail]) if parts else idx
        if cls.mode == "record":
            cls.store.setdefault(layer_idx, []).append(idx.detach().clone())
            return idx
        if cls.mode == "replay":
            c = cls.cursor.get(layer_idx, 0)
            rec = cls.store[layer_idx][c]
            cls.cursor[layer_idx] = c + 1
            if rec.shape != idx.shape:
                raise ValueError(f"routing replay shape mismatch at layer {layer_idx}: {rec.shape} vs {idx.shape}")
            return rec.to(idx.device)
        return idx


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        dx = dy.new_empty((sum(ctx.in_splits),) + tuple(dy.shape[1:]))
        dist.all_to_all_single(dx, dy.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return dx, None, None, None


EXPERT_ROW_ALIGN = 128       # the grouped GEMM walks 128-row tiles; no tile may hold rows of two experts


def padded_expert_layout(expert_of_row: torch.Tensor, num_experts: int, align: int = EXPERT_ROW_ALIGN):
    """Where every row goes in the expert-sorted buffer whose expert groups are padded to ``align`` rows.

    Everything stays on the device (no count is read back): the buffer is sized for the worst case
    ``rows + num_experts * (align - 1)``, unused tiles are marked in the tile map.  Returns ``(order, dest, cap,
    tile_expert, expert_rows)``: ``order`` sorts the rows by expert (stable), ``dest[i]`` is the buffer row of sorted
    position ``i``, ``tile_expert`` (int32, one entry per ``align`` rows) names each tile's expert or -1,
    ``expert_rows`` (int32 ``[E + 1]``) are the padded group boundaries."""
    R, dev = expert_of_row.numel(), expert_of_row.device
    # (not torch.bincount: it reads the maximum back to size its output, a host sync that also forbids graph capture)
    counts = torch.zeros(num_experts, dtype=torch.int64, device=dev).index_add_(
        0, expert_of_row, torch.ones(R, dtype=torch.int64, device=dev))
    padded = (counts + (align - 1)) // align * align
    ends_pad = torch.cumsum(padded, 0)
    offs_pad = ends_pad - padded
    offs = torch.cumsum(counts, 0) - counts
    order = torch.argsort(expert_of_row, stable=True)
    e_sorted = expert_of_row[order]
    dest = offs_pad[e_sorted] + (torch.arange(R, device=dev) - offs[e_sorted])
    cap = (R + num_experts * (align - 1) + align - 1) // align * align
    tile_start = torch.arange(cap // align, device=dev) * align
    te = torch.searchsorted(ends_pad, tile_start, right=True)
    tile_expert = torch.where(te < num_experts, te, torch.full_like(te, -1)).to(torch.int32)
    expert_rows = torch.cat([ends_pad.new_zeros(1), ends_pad]).to(torch.int32)
    return order, dest, cap, tile_expert, expert_rows


def grouped_swiglu_mlp(x, expert_of_row, w1, w2, skip_foreign: bool = False):
    """SwiGLU expert MLPs for rows ``x [R, H]`` with (local) expert ids ``expert_of_row [R]``, in the ORIGINAL row
    order: rows are scattered into the padded expert-sorted buffer, the two grouped GEMMs (one launch each for all
    experts) and the activation run on it, and the rows are gathered back.  ``w1 [E, 2F, H]``, ``w2 [E, H, F]``.
    With ``skip_foreign`` rows whose id is outside ``[0, E)`` (experts that live on another rank) are parked in an
    extra bucket whose tiles are marked unused: they cost no math and come back as zeros."""
    E = w1.shape[0]
    if skip_foreign:
        eo = torch.where((expert_of_row >= 0) & (expert_of_row < E), expert_of_row, torch.full_like(expert_of_row, E))
        order, dest, cap, tile_expert, expert_rows = padded_expert_layout(eo, E + 1)
        tile_expert = torch.where(tile_expert == E, torch.full_like(tile_expert, -1), tile_expert)
        expert_rows = expert_rows[:E + 1].contiguous()
    else:
        order, dest, cap, tile_expert, expert_rows = padded_expert_layout(expert_of_row, E)
    xp = x.new_zeros(cap, x.shape[1]).index_copy(0, dest, x.index_select(0, order))
    a = ops.swiglu(ops.grouped_linear(xp, w1, tile_expert, expert_rows))
    yp = ops.grouped_linear(a, w2, tile_expert, expert_rows)
    inv = torch.empty_like(order)
    inv[order] = dest                       # buffer row of every original row
    return yp.index_select(0, inv)


def route_tokens(logits, cfg, bias=None):
    """``(weights [T, k], indices [T, k], scores [T, E])``.  Softmax routing is the fused top-k op.  Sigmoid routing
    (DeepSeek-V3, GLM4-MoE): experts are *selected* on ``sigmoid(logits) + bias`` but *weighted* by the plain sigmoid
    scores, renormalised over the selected set and multiplied by the routed scaling factor.  (Group-limited
    selection, ``n_group`` / ``topk_group``, is not implemented: all experts form one group.)"""
    if cfg.moe_router_score == "softmax":
        w, idx, probs = ops.topk_router(logits, cfg.moe_top_k, cfg.moe_router_norm_topk_prob)
        return (w * cfg.moe_routed_scaling_factor if cfg.moe_routed_scaling_factor != 1.0 else w), idx, probs
    scores = torch.sigmoid(logits.float())
    sel = scores if bias is None else scores + bias.float()[None, :]
    idx = sel.topk(cfg.moe_top_k, dim=-1).indices
    w = scores.gather(-1, idx)
    if cfg.moe_router_norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * cfg.moe_routed_scaling_factor, idx, scores


class MoEMLP(nn.Module):
    def __init__(self, cfg, ps: ParallelState, dtype, device, gen, layer_idx: int):
        super().__init__()
        self.cfg, self.ps, self.layer_idx = cfg, ps, layer_idx
        E, F, H = cfg.num_experts, cfg.moe_ffn_hidden_size, cfg.hidden_size
        ep = ps.ep.size
        assert E % ep == 0
        self.e_local = E // ep
        self.e_start = ps.ep.rank * self.e_local
        self.router = nn.Module()
        self.router.weight = nn.Parameter(gen.draw(f"layers.{layer_idx}.router", (E, H), 0.02).to(dtype))
        w1 = gen.draw(f"layers.{layer_idx}.experts.fc1", (E, 2 * F, H), 0.02)
        w2 = gen.draw(f"layers.{layer_idx}.experts.fc2", (E, H, F), 0.02 / math.sqrt(2 * cfg.num_layers))
        self.experts = nn.Module()
        self.experts.linear_fc1 = nn.Module()
        self.experts.linear_fc2 = nn.Module()
        sl = slice(self.e_start, self.e_start + self.e_local)
        self.experts.linear_fc1.weight = nn.Parameter(w1[sl].to(dtype).contiguous())
        self.experts.linear_fc2.weight = nn.Parameter(w2[sl].to(dtype).contiguous())
        self.last_aux = None
        self.last_counts = None
        if cfg.moe_router_bias:
            # selection-only bias: no gradient; moved by update_router_bias() towards an even load
            self.router.expert_bias = nn.Parameter(torch.zeros(E, dtype=dtype, device=device), requires_grad=False)
            self._bias_fp32 = torch.zeros(E, dtype=torch.float32, device=device)
        Fs = cfg.moe_shared_expert_ffn
        if Fs > 0:
            self.shared_experts = nn.Module()
            self.shared_experts.linear_fc1 = nn.Module()
            self.shared_experts.linear_fc2 = nn.Module()
            self.shared_experts.linear_fc1.weight = nn.Parameter(
                gen.draw(f"layers.{layer_idx}.shared.fc1", (2 * Fs, H), 0.02).to(device=device, dtype=dtype))
            self.shared_experts.linear_fc2.weight = nn.Parameter(
                gen.draw(f"layers.{layer_idx}.shared.fc2", (H, Fs), 0.02 / math.sqrt(2 * cfg.num_layers)).to(device=device, dtype=dtype))
            if cfg.moe_shared_expert_gate:
                self.shared_experts.gate_weight = nn.Parameter(
                    gen.draw(f"layers.{layer_idx}.shared.gate", (1, H), 0.02).to(device=device, dtype=dtype))

    @torch.no_grad()
    def update_router_bias(self, rate: float = 1e-3, group=None):
        """Auxiliary-loss-free balancing: after a step, raise the bias of experts that got fewer tokens than the
        mean and lower the others by ``rate`` (token counts summed over ``group`` when given)."""
        if self.last_counts is None or not self.cfg.moe_router_bias:
            return
        c = self.last_counts.float()
        if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(c, group=group)
        self._bias_fp32 = self._bias_fp32.to(c.device) + rate * torch.sign(c.mean() - c)
        self.router.expert_bias.copy_(self._bias_fp32)
        self.last_counts = None

    def _shared(self, x):
        se = self.shared_experts
        y = ops.linear(ops.swiglu(ops.linear(x, se.linear_fc1.weight)), se.linear_fc2.weight)
        if hasattr(se, "gate_weight"):
            y = y * torch.sigmoid(ops.linear(x, se.gate_weight).float()).to(y.dtype)
        return y

    def forward(self, x):
        """x ``[T_local, H]`` (the sequence-parallel shard: MoE runs with TP=1 for
        experts, tokens stay sharded)."""
        cfg, ps = self.cfg, self.ps
        T, H = x.shape
        k, E = cfg.moe_top_k, cfg.num_experts
        logits = torch.nn.functional.linear(x.float(), self.router.weight.float())
        w, idx, probs = route_tokens(logits, cfg, self.router.expert_bias if cfg.moe_router_bias else None)
        replay_idx = RoutingReplay.route(self.layer_idx, idx)
        if replay_idx is not idx:
            idx = replay_idx
            w = probs.gather(-1, idx)
            if cfg.moe_router_norm_topk_prob:
                w = w / w.sum(-1, keepdim=True)
            w = w * cfg.moe_routed_scaling_factor
        if cfg.moe_aux_loss_coef > 0 and self.training:
            f = torch.zeros(E, device=x.device).index_add_(0, idx.reshape(-1), torch.ones(T * k, device=x.device))
            self.last_aux = cfg.moe_aux_loss_coef * E * ((f / (T * k)) * probs.mean(0)).sum()

        flat_e = idx.reshape(-1)                      # [T*k]
        order = torch.argsort(flat_e, stable=True)    # permutation: sorted by expert
        src_tok = order // k
        xp = x[src_tok]                               # permuted copies [T*k, H]
        counts = torch.bincount(flat_e, minlength=E)  # tokens per (global) expert
        if cfg.moe_router_bias and self.training:
            self.last_counts = counts.detach() if self.last_counts is None else self.last_counts + counts.detach()

        comm = getattr(self, "ep_comm", None) if x.is_cuda else None
        if ps.ep.size > 1 and comm is not None:
            # dispatch / combine by peer stores into the expert owners' buffers (parallel/ep_peer.py)
            from ..parallel.ep_peer import peer_all_to_all

            ep = ps.ep.size
            allc = comm.exchange_counts(counts).view(ep, ep, self.e_local)          # [src][dst][local expert]
            matrix = allc.sum(-1).tolist()
            recv_counts = allc[:, ps.ep.rank, :]
            xr = peer_all_to_all(xp, matrix, comm)
            rc = recv_counts.reshape(-1)
            seg_expert = torch.arange(self.e_local, device=x.device).repeat(ep)
            ye = grouped_swiglu_mlp(xr, torch.repeat_interleave(seg_expert, rc), self.experts.linear_fc1.weight,
                                    self.experts.linear_fc2.weight)
            yp = peer_all_to_all(ye, [[matrix[d][s_] for d in range(ep)] for s_ in range(ep)], comm)
        elif ps.ep.size > 1:
            ep = ps.ep.size
            send_counts = counts.view(ep, self.e_local)
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=ps.ep.group)
            in_splits = send_counts.sum(1).tolist()
            out_splits = recv_counts.sum(1).tolist()
            xr = _AllToAll.apply(xp, out_splits, in_splits, ps.ep.group)
            # received rows are ordered (src rank, local expert); regroup by local expert
            rc = recv_counts.reshape(-1)
            seg_expert = torch.arange(self.e_local, device=x.device).repeat(ep)
            row_expert = torch.repeat_interleave(seg_expert, rc)
            yr = grouped_swiglu_mlp(xr, row_expert, self.experts.linear_fc1.weight, self.experts.linear_fc2.weight)
            yp = _AllToAll.apply(yr, in_splits, out_splits, ps.ep.group)
        else:
            # rows of ``xp`` are already sorted by expert; the grouped path re-derives the (padded) layout on the
            # device, so no count leaves the GPU
            yp = grouped_swiglu_mlp(xp, flat_e[order], self.experts.linear_fc1.weight, self.experts.linear_fc2.weight)

        wf = w.reshape(-1)[order].to(yp.dtype)
        out = torch.zeros(T, H, dtype=yp.dtype, device=x.device)
        out = out.index_add(0, src_tok, yp * wf[:, None])
        if cfg.moe_shared_expert_ffn > 0:
            out = out + self._shared(x).to(out.dtype)
        return out.to(x.dtype)
