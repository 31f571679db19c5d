"""Gated DeltaNet (GDN) linear attention: the gated delta rule in recurrent and chunked form, and the mixer layer
of the Qwen3-Next family built on it.

The reference reaches this op through Megatron's GDN layer and the ``fla`` Triton kernels
(relax/backends/megatron/model.py GDN context-parallel patch :357-644; weight names in
relax/backends/megatron/weight_conversion/qwen3_next.py).  Here the op is plain PyTorch - correct, differentiable,
chunk-parallel (all chunk-local work is batched matmuls; only the ``[dk, dv]`` state walks the chunks) - and runs on
whichever device holds the tensors.  There is no hand-written sm_100a kernel for it yet.

Per head, with state ``S [dk, dv]``, decay ``a_t = exp(g_t)`` (``g_t <= 0``) and write strength ``beta_t``::

    S_t = a_t S_{t-1} + beta_t k_t (v_t - (a_t S_{t-1})^T k_t)^T        o_t = S_t^T q_t
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


def gated_delta_rule_recurrent(q, k, v, g, beta, state: Optional[torch.Tensor] = None):
    """Token-by-token oracle.  ``q, k [T, H, dk]``, ``v [T, H, dv]``, ``g, beta [T, H]``.  ``q`` is scaled by
    ``dk ** -0.5`` inside.  Returns ``(o [T, H, dv], final_state [H, dk, dv])`` in fp32."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    q, k, v, g, beta = (x.float() for x in (q, k, v, g, beta))
    q = q * dk ** -0.5
    S = torch.zeros(H, dk, dv, device=q.device) if state is None else state.float().clone()
    out = []
    for t in range(T):
        S = S * g[t].exp()[:, None, None]
        pred = torch.einsum("hkv,hk->hv", S, k[t])
        u = (v[t] - pred) * beta[t][:, None]
        S = S + torch.einsum("hk,hv->hkv", k[t], u)
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out) if out else q.new_zeros(0, H, dv), S


def gated_delta_rule_chunked(q, k, v, g, beta, chunk: int = 64, state: Optional[torch.Tensor] = None):
    """Same function, chunk-parallel.  Inside a chunk the writes ``u_i`` obey a unit-lower-triangular system
    ``(I + L) U = beta V - (beta K e^gamma) S_0`` with ``L_ij = beta_i (k_i . k_j) e^(gamma_i - gamma_j)`` for
    ``j < i`` (``gamma`` = running sum of ``g`` inside the chunk); it is solved once per chunk for both right-hand
    sides, after which output and state update are matmuls."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    q, k, v, g, beta = (x.float() for x in (q, k, v, g, beta))
    q = q * dk ** -0.5
    pad = (-T) % chunk
    if pad:
        z = lambda x: F.pad(x, (0, 0) * (x.dim() - 1) + (0, pad))
        q, k, v, g, beta = z(q), z(k), z(v), z(g), z(beta)     # padded steps: g = 0, beta = 0 -> state untouched
    n = (T + pad) // chunk
    # [H, n, C, d]
    hs = lambda x: x.reshape(n, chunk, H, -1).permute(2, 0, 1, 3)
    q, k, v = hs(q), hs(k), hs(v)
    g = g.reshape(n, chunk, H).permute(2, 0, 1)
    beta = beta.reshape(n, chunk, H).permute(2, 0, 1)
    gamma = g.cumsum(-1)                                       # [H, n, C]
    diff = gamma[..., :, None] - gamma[..., None, :]           # gamma_i - gamma_j
    tril = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device))
    D = torch.where(tril, diff, torch.full_like(diff, -float("inf"))).exp()     # 0 above the diagonal
    kb = k * beta[..., None]
    L = (kb @ k.transpose(-1, -2)) * D
    L = L.masked_fill(torch.triu(torch.ones_like(tril)), 0.0)  # strictly lower
    eye = torch.eye(chunk, device=q.device).expand_as(L)
    Tm = torch.linalg.solve_triangular(eye + L, eye, upper=False)
    u_own = Tm @ (v * beta[..., None])                         # writes if the incoming state were zero
    k_in = Tm @ (kb * gamma.exp()[..., None])                  # how the incoming state changes the writes
    qk = (q @ k.transpose(-1, -2)) * D                         # causal, decayed (diagonal included)
    S = torch.zeros(H, dk, dv, device=q.device) if state is None else state.float().clone()
    outs = []
    for c in range(n):
        u = u_own[:, c] - k_in[:, c] @ S
        o = (q[:, c] * gamma[:, c].exp()[..., None]) @ S + qk[:, c] @ u
        last = gamma[:, c, -1]
        S = S * last.exp()[:, None, None] + (k[:, c] * (last[:, None] - gamma[:, c]).exp()[..., None]).transpose(-1, -2) @ u
        outs.append(o)
    o = torch.stack(outs, 1).permute(1, 2, 0, 3).reshape(n * chunk, H, dv)
    return o[:T], S


def gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, chunk: int = 64):
    """Packed sequences: the state restarts at every ``cu_seqlens`` boundary."""
    cu = [int(x) for x in cu_seqlens.tolist()]
    outs = [gated_delta_rule_chunked(q[a:b], k[a:b], v[a:b], g[a:b], beta[a:b], chunk)[0] for a, b in zip(cu[:-1], cu[1:]) if b > a]
    tail = q.shape[0] - cu[-1]
    if tail > 0:
        outs.append(q.new_zeros(tail, q.shape[1], v.shape[-1], dtype=torch.float32))
    return torch.cat(outs)


def causal_conv1d_varlen(x, weight, cu_seqlens):
    """Depth-wise causal convolution over tokens that never reads across a sequence boundary.
    ``x [T, C]``, ``weight [C, K]``; output ``[T, C]`` (SiLU applied, as in the mixer)."""
    T, C = x.shape
    K = weight.shape[1]
    cu = cu_seqlens.to(torch.int64)
    rows = torch.arange(T, device=x.device)
    seq = torch.bucketize(rows, cu[1:], right=True).clamp_max(cu.numel() - 2)
    start = cu[:-1][seq]
    y = torch.zeros_like(x, dtype=torch.float32)
    for j in range(K):                     # tap j looks back K-1-j tokens
        back = K - 1 - j
        src = rows - back
        ok = (src >= start)[:, None]
        y = y + torch.where(ok, x[src.clamp_min(0)].float(), torch.zeros((), device=x.device)) * weight[:, j].float()
    return F.silu(y).to(x.dtype)


class GatedDeltaNet(nn.Module):
    """The GDN token mixer: ``in_proj_qkvz`` / ``in_proj_ba`` -> causal depth-wise conv + SiLU on q, k, v ->
    L2-normalised q, k; ``beta = sigmoid(b)``; ``g = -exp(A_log) * softplus(a + dt_bias)`` -> gated delta rule ->
    RMSNorm gated by ``silu(z)`` -> ``out_proj``.  ``num_v_heads`` may be a multiple of ``num_k_heads`` (keys and
    queries are shared by the value heads of a group)."""

    def __init__(self, hidden_size: int, num_k_heads: int, num_v_heads: int, head_k_dim: int, head_v_dim: int,
                 conv_kernel: int = 4, eps: float = 1e-6, dtype=torch.float32, device="cpu", seed: int = 0, chunk: int = 64):
        super().__init__()
        assert num_v_heads % num_k_heads == 0
        self.hk, self.hv, self.dk, self.dv, self.eps, self.chunk = num_k_heads, num_v_heads, head_k_dim, head_v_dim, eps, chunk
        gen = torch.Generator().manual_seed(seed)
        kd, vd = num_k_heads * head_k_dim, num_v_heads * head_v_dim
        mk = lambda *s, std=0.02: nn.Parameter((torch.randn(*s, generator=gen) * std).to(device=device, dtype=dtype))
        self.in_proj_qkvz = nn.Module()
        self.in_proj_qkvz.weight = mk(2 * kd + 2 * vd, hidden_size)
        self.in_proj_ba = nn.Module()
        self.in_proj_ba.weight = mk(2 * num_v_heads, hidden_size)
        self.conv1d = nn.Module()
        self.conv1d.weight = mk(2 * kd + vd, conv_kernel, std=0.3)
        self.dt_bias = nn.Parameter(torch.ones(num_v_heads, dtype=dtype, device=device))
        self.A_log = nn.Parameter(torch.log(torch.empty(num_v_heads).uniform_(1, 16, generator=gen)).to(device=device, dtype=dtype))
        self.norm = nn.Module()
        self.norm.weight = nn.Parameter(torch.ones(head_v_dim, dtype=dtype, device=device))
        self.out_proj = nn.Module()
        self.out_proj.weight = mk(hidden_size, vd)

    def forward(self, x, cu_seqlens, recurrent: bool = False):
        T = x.shape[0]
        kd, vd = self.hk * self.dk, self.hv * self.dv
        qkvz = ops.linear(x, self.in_proj_qkvz.weight)
        ba = ops.linear(x, self.in_proj_ba.weight).float()
        qkv, z = qkvz[:, : 2 * kd + vd], qkvz[:, 2 * kd + vd:]
        qkv = causal_conv1d_varlen(qkv, self.conv1d.weight, cu_seqlens)
        q = F.normalize(qkv[:, :kd].reshape(T, self.hk, self.dk).float(), dim=-1)
        k = F.normalize(qkv[:, kd:2 * kd].reshape(T, self.hk, self.dk).float(), dim=-1)
        v = qkv[:, 2 * kd:].reshape(T, self.hv, self.dv)
        rep = self.hv // self.hk
        if rep > 1:
            q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
        beta = torch.sigmoid(ba[:, : self.hv])
        g = -self.A_log.float().exp() * F.softplus(ba[:, self.hv:] + self.dt_bias.float())
        if recurrent:
            cu = [int(c) for c in cu_seqlens.tolist()]
            o = torch.cat([gated_delta_rule_recurrent(q[a:b], k[a:b], v[a:b], g[a:b], beta[a:b])[0] for a, b in zip(cu[:-1], cu[1:])])
        else:
            o = gated_delta_rule_varlen(q, k, v, g, beta, cu_seqlens, self.chunk)
        o = ops.rmsnorm(o.to(x.dtype), self.norm.weight, self.eps) * F.silu(z.reshape(T, self.hv, self.dv))
        return ops.linear(o.reshape(T, vd), self.out_proj.weight)
