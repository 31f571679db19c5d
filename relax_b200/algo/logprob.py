"""Vocab-parallel log-prob / entropy from logits (eager oracle).

The production path never materialises ``[T, V]`` logits: it is the fused
LM-head kernel in :mod:`relax_b200.ops.fused_lm_head`.  This module is the
plain-PyTorch statement of the same maths, used on CPU, in tests and as the
unfused baseline.  Parity target: relax/utils/training/ppo_utils.py:480-629
(three/four tensor-parallel all-reduces: MAX, SUM exp, SUM target logit,
SUM p*z) and relax/backends/megatron/loss.py:290-463.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _ar(t, op, group):
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=op, group=group)
    return t


class _VocabParallelLogProbEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, group, vocab_start, with_entropy):
        # logits: [T, V_local] (any float dtype), targets: [T] global ids
        z = logits.float()
        v_local = z.shape[-1]
        m = _ar(z.max(-1).values, dist.ReduceOp.MAX, group)
        z = z - m[:, None]
        e = torch.exp(z)
        s = _ar(e.sum(-1), dist.ReduceOp.SUM, group)
        local_t = targets - vocab_start
        in_range = (local_t >= 0) & (local_t < v_local)
        safe_t = torch.where(in_range, local_t, torch.zeros_like(local_t))
        zt = torch.where(in_range, z.gather(-1, safe_t[:, None])[:, 0], torch.zeros_like(m))
        zt = _ar(zt, dist.ReduceOp.SUM, group)
        log_s = torch.log(s)
        logp = zt - log_s
        p = e / s[:, None]
        if with_entropy:
            pz = _ar((p * z).sum(-1), dist.ReduceOp.SUM, group)
            ent = log_s - pz
        else:
            pz = torch.zeros_like(m)
            ent = torch.zeros_like(m)
        ctx.save_for_backward(p, z, pz, safe_t, in_range)
        ctx.with_entropy = with_entropy
        ctx.in_dtype = logits.dtype
        return logp, ent

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        p, z, pz, safe_t, in_range = ctx.saved_tensors
        # d logp / d z_j = onehot_j - p_j
        grad = -p * g_logp[:, None]
        grad.scatter_add_(-1, safe_t[:, None], (g_logp * in_range)[:, None].to(grad.dtype))
        if ctx.with_entropy and g_ent is not None:
            # d H / d z_j = p_j * (sum_k p_k z_k - z_j)
            grad = grad + (p * (pz[:, None] - z)) * g_ent[:, None]
        return grad.to(ctx.in_dtype), None, None, None, None


def vocab_parallel_log_probs_and_entropy(
    logits: torch.Tensor,
    targets: torch.Tensor,
    tp_group=None,
    vocab_start: int = 0,
    with_entropy: bool = True,
    temperature: float = 1.0,
):
    """Return ``(log_prob[T], entropy[T])`` in fp32 for a vocab shard."""
    if temperature != 1.0:
        logits = logits / temperature
    return _VocabParallelLogProbEntropy.apply(logits, targets, tp_group, vocab_start, with_entropy)


def chunked_log_probs_and_entropy(hidden, weight, targets, tp_group=None, vocab_start=0, with_entropy=True,
                                  temperature: float = 1.0, chunk_size: int = 4096):
    """LM head + log-prob over token chunks so at most ``chunk_size x V_local``
    logits exist at once (the role of ``--log-probs-chunk-size``)."""
    lps, ents = [], []
    # a rank may hold no rows at all (context parallelism: the response can sit wholly on the other ranks); it
    # still runs one empty chunk so the tensor-parallel collectives inside match and the graph reaches the weights
    for s in range(0, max(1, hidden.shape[0]), chunk_size):
        h = hidden[s : s + chunk_size]
        logits = h @ weight.t()
        lp, en = vocab_parallel_log_probs_and_entropy(
            logits, targets[s : s + chunk_size], tp_group, vocab_start, with_entropy, temperature
        )
        lps.append(lp)
        ents.append(en)
    return torch.cat(lps), torch.cat(ents)


def top_k_log_probs_on_ids(logits, ids, tp_group=None, vocab_start: int = 0):
    """log-softmax evaluated at given candidate ids ``[T, K]`` of a vocab shard
    (teacher top-k for on-policy distillation; relax/utils/opd/opd_utils.py:1023-1095)."""
    z = logits.float()
    v_local = z.shape[-1]
    m = _ar(z.max(-1).values, dist.ReduceOp.MAX, tp_group)
    s = _ar(torch.exp(z - m[:, None]).sum(-1), dist.ReduceOp.SUM, tp_group)
    loc = ids - vocab_start
    ok = (loc >= 0) & (loc < v_local)
    g = torch.where(ok, z.gather(-1, torch.where(ok, loc, torch.zeros_like(loc))), torch.zeros((), dtype=z.dtype))
    g = _ar(g, dist.ReduceOp.SUM, tp_group)
    return g - m[:, None] - torch.log(s)[:, None]
