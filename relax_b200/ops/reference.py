"""Plain-PyTorch statements of every hot operator.

These are (1) the CPU path, (2) the fp32 oracle every CUDA kernel is tested
against and (3) the unfused library baseline the fused kernels are timed
against.  They run through autograd, so they need no hand-written backward.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

# --------------------------------------------------------------------------- norms / activations


def rmsnorm(x, w, eps: float = 1e-6):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype)


def add_rmsnorm(x, residual, w, eps: float = 1e-6):
    """``r = x + residual; y = rmsnorm(r)``; returns ``(y, r)``."""
    r = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(r, w, eps), r


def swiglu(gate_up):
    g, u = gate_up.chunk(2, dim=-1)
    return (F.silu(g.float()) * u.float()).to(gate_up.dtype)


def linear(x, w, bias=None):
    return F.linear(x, w, bias)


# --------------------------------------------------------------------------- rotary embedding


def rope_cos_sin(positions, head_dim: int, theta: float, mrope_section=None):
    """cos/sin tables ``[T, head_dim/2]`` (fp32).  ``positions`` is ``[T]`` or,
    for multimodal M-RoPE, ``[3, T]`` (temporal, height, width) with
    ``mrope_section`` giving how many of the ``head_dim/2`` frequencies follow
    each of the three position streams."""
    half = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, device=positions.device, dtype=torch.float32) / half))
    if positions.dim() == 1:
        ang = positions.float()[:, None] * inv[None, :]
    else:
        assert mrope_section is not None and sum(mrope_section) == half
        ang3 = positions.float()[:, :, None] * inv[None, None, :]  # [3, T, half]
        parts, s = [], 0
        for i, n in enumerate(mrope_section):
            parts.append(ang3[i, :, s : s + n])
            s += n
        ang = torch.cat(parts, -1)
    return ang.cos(), ang.sin()


def apply_rope(x, cos, sin):
    """Rotate-half (NeoX) convention on ``x[T, H, D]``."""
    d = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :d], xf[..., d:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)


# --------------------------------------------------------------------------- attention


def attention_varlen(q, k, v, cu_seqlens, causal: bool = True, scale: Optional[float] = None,
                     cu_seqlens_k=None, return_lse: bool = False):
    """Packed variable-length attention.  q ``[Tq, Hq, D]``, k/v ``[Tk, Hkv, D]``;
    sequence ``i`` owns rows ``cu[i]:cu[i+1]``.  With ``causal`` the last query
    of a sequence is aligned with its last key (bottom-right alignment), so a
    shorter query block attends to a longer key prefix correctly."""
    Hq, Hkv, D = q.shape[1], k.shape[1], q.shape[2]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    cu_q = cu_seqlens.tolist()
    cu_k = (cu_seqlens_k if cu_seqlens_k is not None else cu_seqlens).tolist()
    outs, lses = [], []
    for i in range(len(cu_q) - 1):
        qs = q[cu_q[i] : cu_q[i + 1]].float().transpose(0, 1)  # [Hq, Lq, D]
        ks = k[cu_k[i] : cu_k[i + 1]].float().transpose(0, 1).repeat_interleave(g, 0)
        vs = v[cu_k[i] : cu_k[i + 1]].float().transpose(0, 1).repeat_interleave(g, 0)
        s = torch.einsum("hqd,hkd->hqk", qs, ks) * scale
        if causal:
            Lq, Lk = qs.shape[1], ks.shape[1]
            qi = torch.arange(Lq, device=q.device)[:, None] + (Lk - Lq)
            ki = torch.arange(Lk, device=q.device)[None, :]
            s = s.masked_fill(ki > qi, float("-inf"))
        lse = torch.logsumexp(s, -1)
        p = torch.exp(s - lse[..., None])
        outs.append(torch.einsum("hqk,hkd->hqd", p, vs).transpose(0, 1))
        lses.append(lse.transpose(0, 1))
    o = torch.cat(outs, 0).to(q.dtype)
    if return_lse:
        return o, torch.cat(lses, 0)
    return o


def paged_decode_attention(q, k_cache, v_cache, block_tables, context_lens, scale: Optional[float] = None):
    """One query token per sequence against a paged KV cache.

    q ``[B, Hq, D]``; caches ``[num_blocks, block_size, Hkv, D]``;
    ``block_tables [B, max_blocks]`` int32; ``context_lens [B]`` (including the
    current token, whose K/V must already be in the cache)."""
    B, Hq, D = q.shape
    bs, Hkv = k_cache.shape[1], k_cache.shape[2]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    for b in range(B):
        L = int(context_lens[b])
        nb = (L + bs - 1) // bs
        blocks = block_tables[b, :nb].long()
        ks = k_cache[blocks].reshape(-1, Hkv, D)[:L].float()
        vs = v_cache[blocks].reshape(-1, Hkv, D)[:L].float()
        qq = q[b].float().view(Hkv, g, D)
        s = torch.einsum("hgd,lhd->hgl", qq, ks) * scale
        p = torch.softmax(s, -1)
        out[b] = torch.einsum("hgl,lhd->hgd", p, vs).reshape(Hq, D).to(q.dtype)
    return out


# --------------------------------------------------------------------------- sampling / routing


def sample(logits, temperature, top_k, top_p, uniform):
    """Sample one token per row.  ``temperature/top_k/top_p`` are per-row tensors
    (top_k <= 0 disables, top_p >= 1 disables); ``uniform [B]`` are U(0,1)
    draws supplied by the caller so the op is deterministic.  Returns
    ``(token[B], log_prob[B])`` where the log-prob is that of the *unfiltered*
    temperature-scaled distribution (what the trainer recomputes)."""
    z = logits.float() / temperature.float().clamp_min(1e-6)[:, None]
    logp_full = torch.log_softmax(z, -1)
    greedy = temperature <= 0
    V = z.shape[-1]
    # kept set: the k largest, then the shortest prefix (descending order) of those whose
    # renormalised mass reaches top_p
    sorted_z, idx = torch.sort(z, -1, descending=True)
    ranks = torch.arange(V, device=z.device)[None, :]
    k = torch.where(top_k > 0, top_k, torch.full_like(top_k, V))
    keep = ranks < k[:, None]
    probs = torch.softmax(sorted_z.masked_fill(~keep, float("-inf")), -1)
    csum = torch.cumsum(probs, -1)
    keep &= (csum - probs) < top_p.float()[:, None]
    mask = torch.zeros_like(keep).scatter(-1, idx, keep)
    # inverse CDF in vocabulary order over the kept entries
    e = torch.exp(z - z.max(-1, keepdim=True).values) * mask
    c = torch.cumsum(e.double(), -1)
    target = uniform.double()[:, None] * c[:, -1:]
    pick = (c <= target).sum(-1).clamp_max(V - 1)
    # rounding at the end of the CDF must not select a filtered slot
    last_kept = (mask * torch.arange(V, device=z.device)[None, :]).amax(-1)
    tok = torch.minimum(pick, last_kept)
    tok = torch.where(greedy, z.argmax(-1), tok)
    return tok, logp_full.gather(-1, tok[:, None])[:, 0]


def grouped_linear(x, w, tile_expert, expert_rows):
    """``y[row] = x[row] @ w[e].T`` for the rows of expert ``e`` (``expert_rows[e] : expert_rows[e + 1]`` of the padded,
    expert-sorted buffer); rows outside every expert's range stay zero."""
    y = x.new_zeros(x.shape[0], w.shape[1])
    bounds = expert_rows.tolist()
    parts = []
    for e in range(w.shape[0]):
        a, b = bounds[e], bounds[e + 1]
        parts.append(x[a:b] @ w[e].t().to(x.dtype))
    tail = x.new_zeros(x.shape[0] - bounds[w.shape[0]], w.shape[1]) + 0.0 * w.sum().to(x.dtype)
    return torch.cat(parts + [tail]) if parts else y


def decode_advance(tok_new, lp_new, st, block_size: int):
    """Turn the tokens sampled by one decode step into the next step's inputs, in place, without the host.

    ``st`` holds the batch state, one entry per row: ``tok`` (next input token), ``pos`` (its position), ``ctx``
    (context length including it), ``slots`` (its KV-cache row), ``bt`` (block table ``[B, max_blocks]``), ``active``
    (0 once the row stopped), ``remain`` (tokens it may still emit), ``eos`` (-1: none), ``stop`` (``[B, n]`` extra
    stop ids, -1 padding); the window ring ``out_tok`` / ``out_lp`` ``[W, B]`` with its write index ``counter``; the
    uniform draws of the whole window ``u_all [W, B]`` and of the coming step ``u [B]``.  Rows that already stopped
    append -1 and change nothing."""
    c = int(st["counter"][0])
    W = st["out_tok"].shape[0]
    if c >= W:
        return
    act = st["active"] != 0
    st["out_tok"][c] = torch.where(act, tok_new, torch.full_like(tok_new, -1))
    st["out_lp"][c] = torch.where(act, lp_new, torch.zeros_like(lp_new))
    left = st["remain"] - act.to(st["remain"].dtype)
    stop = (st["eos"] >= 0) & (tok_new == st["eos"])
    if st["stop"].shape[1]:
        stop = stop | ((st["stop"] >= 0) & (st["stop"] == tok_new[:, None])).any(-1)
    p = st["pos"] + 1
    blk = p // block_size
    fits = blk < st["bt"].shape[1]
    go = act & ~stop & (left > 0) & fits
    new_slot = st["bt"].gather(1, blk.clamp_max(st["bt"].shape[1] - 1)[:, None].long())[:, 0].long() * block_size + p % block_size
    st["tok"].copy_(torch.where(go, tok_new, st["tok"]))
    st["pos"].copy_(torch.where(go, p, st["pos"]))
    st["ctx"].copy_(torch.where(go, (p + 1).to(st["ctx"].dtype), st["ctx"]))
    st["slots"].copy_(torch.where(go, new_slot, st["slots"]))
    st["active"].copy_((go).to(st["active"].dtype))
    st["remain"].copy_(left)
    if c + 1 < W:
        st["u"].copy_(st["u_all"][c + 1])
    st["counter"] += 1


def topk_router(logits, top_k: int, norm_topk_prob: bool = True):
    """fp32 softmax over experts then top-k; returns ``(weights[T,k], idx[T,k], probs[T,E])``."""
    p = torch.softmax(logits.float(), -1)
    w, idx = torch.topk(p, top_k, dim=-1)
    if norm_topk_prob:
        w = w / w.sum(-1, keepdim=True)
    return w, idx, p


# --------------------------------------------------------------------------- optimizer


def adam_step(p32, g, m, v, step: int, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
              grad_scale: float = 1.0):
    """AdamW on fp32 master weights (decoupled decay, bias correction)."""
    gf = g.float() * grad_scale
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    bc1 = 1 - beta1**step
    bc2 = 1 - beta2**step
    denom = (v / bc2).sqrt_().add_(eps)
    p32.mul_(1 - lr * weight_decay).addcdiv_(m / bc1, denom, value=-lr)
    return p32


# --------------------------------------------------------------------------- quantisers


def fake_int4_quant(x, block_m: int, block_n: int, sym: bool = True):
    """Group-wise int4 fake quantisation.  Groups are ``block_m x block_n`` tiles
    of the 2-D input.  Symmetric: ``scale = absmax/7``, q in [-8, 7] (round to
    nearest even); asymmetric: ``scale = (max-min)/15`` with an integer
    zero-point, q in [0, 15].  Returns ``(dequantised, scale, zero)`` in the
    input dtype; scale/zero have one entry per group."""
    M, N = x.shape
    gm, gn = (M + block_m - 1) // block_m, (N + block_n - 1) // block_n
    xp = x.float()
    if M % block_m or N % block_n:
        xp = F.pad(xp, (0, gn * block_n - N, 0, gm * block_m - M))
    t = xp.view(gm, block_m, gn, block_n).permute(0, 2, 1, 3).reshape(gm, gn, -1)
    valid = torch.ones(gm * block_m, gn * block_n, dtype=torch.bool, device=x.device)
    valid[M:, :] = False
    valid[:, N:] = False
    vm = valid.view(gm, block_m, gn, block_n).permute(0, 2, 1, 3).reshape(gm, gn, -1)
    if sym:
        amax = torch.where(vm, t.abs(), torch.zeros_like(t)).amax(-1)
        scale = (amax / 7.0).clamp_min(1e-5)
        q = torch.round(t / scale[..., None]).clamp(-8, 7)
        dq = q * scale[..., None]
        zero = torch.zeros_like(scale)
    else:
        tmax = torch.where(vm, t, torch.full_like(t, -float("inf"))).amax(-1)
        tmin = torch.where(vm, t, torch.full_like(t, float("inf"))).amin(-1)
        scale = ((tmax - tmin) / 15.0).clamp_min(1e-5)
        zero = torch.round(-tmin / scale).clamp(0, 15)
        q = (torch.round(t / scale[..., None]) + zero[..., None]).clamp(0, 15)
        dq = (q - zero[..., None]) * scale[..., None]
    out = dq.view(gm, gn, block_m, block_n).permute(0, 2, 1, 3).reshape(gm * block_m, gn * block_n)[:M, :N]
    return out.to(x.dtype), scale.to(x.dtype), zero.to(x.dtype)


FP8_E4M3_MAX = 448.0


def blockwise_cast_to_fp8(w, block: int = 128, ue8m0: bool = False):
    """Per ``block x block`` absmax scaling to e4m3.  Returns ``(w_fp8, scale_inv)``
    with ``w ~= w_fp8 * scale_inv[block]``; ``ue8m0`` rounds the scale up to a
    power of two (the MX-style exponent-only scale format)."""
    M, N = w.shape
    gm, gn = (M + block - 1) // block, (N + block - 1) // block
    wp = F.pad(w.float(), (0, gn * block - N, 0, gm * block - M))
    t = wp.view(gm, block, gn, block)
    amax = t.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / FP8_E4M3_MAX
    if ue8m0:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = (t / scale[:, None, :, None]).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX)
    q = q.reshape(gm * block, gn * block)[:M, :N].to(torch.float8_e4m3fn)
    return q, scale


def blockwise_dequant_fp8(q, scale_inv, block: int = 128, dtype=torch.bfloat16):
    M, N = q.shape
    s = scale_inv.repeat_interleave(block, 0)[:M].repeat_interleave(block, 1)[:, :N]
    return (q.float() * s).to(dtype)
