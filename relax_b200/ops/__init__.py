"""Operator entry points.

CUDA tensors go to the hand-written sm_100a kernels in the in-tree extension
(:mod:`relax_b200.ops.cuda`); CPU tensors go to the PyTorch statements in
:mod:`relax_b200.ops.reference`.  There is no silent fallback on a GPU: if the
extension is missing, a CUDA call raises.  ``RELAX_B200_FORCE_REFERENCE=1``
routes CUDA tensors through the PyTorch/library path on purpose - that is the
"unfused NCCL + cuBLAS" baseline arm used for A/B timing.
"""
from __future__ import annotations

import torch

import os

from . import reference as ref


def _force_ref() -> bool:
    return os.environ.get("RELAX_B200_FORCE_REFERENCE", "0") == "1"


def _use_cuda(t) -> bool:
    return t.is_cuda and not _force_ref()


def _cuda():
    from . import cuda as _c

    return _c


def _vec_ok(t) -> bool:
    """Rows of ``t`` split into 16-byte vectors (what the elementwise kernels load)."""
    return t.shape[-1] % (16 // t.element_size()) == 0


def rmsnorm(x, w, eps=1e-6):
    return _cuda().rmsnorm(x, w, eps) if _use_cuda(x) and _vec_ok(x) else ref.rmsnorm(x, w, eps)


def add_rmsnorm(x, residual, w, eps=1e-6):
    if _use_cuda(x) and _vec_ok(x):
        return _cuda().add_rmsnorm(x, residual, w, eps)
    return ref.add_rmsnorm(x, residual, w, eps)


def swiglu(gate_up):
    if _use_cuda(gate_up) and (gate_up.shape[-1] // 2) % (16 // gate_up.element_size()) == 0:
        return _cuda().swiglu(gate_up)
    return ref.swiglu(gate_up)


def linear(x, w, bias=None):
    return _cuda().linear(x, w, bias) if _use_cuda(x) else ref.linear(x, w, bias)


def rope_cos_sin(positions, head_dim, theta, mrope_section=None):
    return ref.rope_cos_sin(positions, head_dim, theta, mrope_section)


_WARNED: set = set()


def _statement_on_gpu(what: str):
    """A shape no sm_100a kernel of this package covers runs as its PyTorch statement on the GPU; said once."""
    if what not in _WARNED:
        _WARNED.add(what)
        import warnings

        warnings.warn(f"relax_b200: {what}: no sm_100a kernel for this shape, running the PyTorch statement", stacklevel=3)


def apply_rope(x, cos, sin):
    if _use_cuda(x):
        if (x.shape[-1] // 2) % (16 // x.element_size()) == 0:
            return _cuda().apply_rope(x, cos, sin)
        _statement_on_gpu(f"rotary width {x.shape[-1]}")
    return ref.apply_rope(x, cos, sin)


def attention_varlen(q, k, v, cu_seqlens, causal=True, scale=None, cu_seqlens_k=None, max_seqlen=None):
    """Packed varlen attention.  On a GPU the tcgen05 kernels take bf16 with head_dim 128; narrower heads
    (64 / 80 / 96 - ViT towers, small models) are zero-padded to 128, which leaves q k^T and the first ``D`` output
    columns unchanged (the softmax scale stays 1 / sqrt(D))."""
    if _use_cuda(q):
        D = q.shape[-1]
        if q.dtype == torch.bfloat16 and D == v.shape[-1] and D <= 128 and D % 8 == 0:
            if D == 128:
                return _cuda().attention_varlen(q, k, v, cu_seqlens, causal, scale, cu_seqlens_k, max_seqlen)
            pad = (0, 128 - D)
            F = torch.nn.functional
            scale = scale if scale is not None else D ** -0.5
            o = _cuda().attention_varlen(F.pad(q, pad), F.pad(k, pad), F.pad(v, pad), cu_seqlens, causal, scale,
                                         cu_seqlens_k, max_seqlen)
            return o[..., :D]
        _statement_on_gpu(f"attention with {q.dtype}, head_dim {D} / {v.shape[-1]}")
    return ref.attention_varlen(q, k, v, cu_seqlens, causal, scale, cu_seqlens_k)


def paged_decode_attention(q, k_cache, v_cache, block_tables, context_lens, scale=None):
    if _use_cuda(q):
        if q.dtype == torch.bfloat16 and q.shape[-1] == 128:
            return _cuda().paged_decode_attention(q, k_cache, v_cache, block_tables, context_lens, scale)
        _statement_on_gpu(f"paged decode attention with {q.dtype}, head_dim {q.shape[-1]}")
    return ref.paged_decode_attention(q, k_cache, v_cache, block_tables, context_lens, scale)


def sample(logits, temperature, top_k, top_p, uniform):
    if _use_cuda(logits):
        return _cuda().sample(logits, temperature, top_k, top_p, uniform)
    return ref.sample(logits, temperature, top_k, top_p, uniform)


def grouped_linear(x, w, tile_expert, expert_rows):
    """Per-expert linear over an expert-sorted token buffer whose expert groups start at multiples of 128 rows
    (see :func:`relax_b200.models.moe.padded_expert_layout`); ``w`` is ``[E, N, K]``."""
    if _use_cuda(x):
        return _cuda().grouped_linear(x, w, tile_expert, expert_rows)
    return ref.grouped_linear(x, w, tile_expert, expert_rows)


def decode_advance(tok_new, lp_new, state, block_size):
    """In-place advance of the rollout engine's device-resident batch state after one decode step."""
    if _use_cuda(tok_new):
        return _cuda().decode_advance(tok_new, lp_new, state, block_size)
    return ref.decode_advance(tok_new, lp_new, state, block_size)


def topk_router(logits, top_k, norm_topk_prob=True):
    if _use_cuda(logits):
        return _cuda().topk_router(logits, top_k, norm_topk_prob)
    return ref.topk_router(logits, top_k, norm_topk_prob)


def fused_lm_head_logprob(hidden, weight, targets, tp_group=None, vocab_start=0, with_entropy=True,
                          temperature=1.0, chunk_size=4096):
    """LM-head GEMM fused with online-softmax log-prob / entropy; ``[T, V]`` is never stored."""
    if _use_cuda(hidden):
        return _cuda().fused_lm_head_logprob(hidden, weight, targets, tp_group, vocab_start, with_entropy, temperature)
    from ..algo.logprob import chunked_log_probs_and_entropy

    return chunked_log_probs_and_entropy(hidden, weight, targets, tp_group, vocab_start, with_entropy,
                                         temperature, chunk_size)


def fake_int4_quant(x, block_m, block_n, sym=True):
    if _use_cuda(x):
        return _cuda().fake_int4_quant(x, block_m, block_n, sym)
    return ref.fake_int4_quant(x, block_m, block_n, sym)


def blockwise_cast_to_fp8(w, block=128, ue8m0=False):
    if _use_cuda(w):
        return _cuda().blockwise_cast_to_fp8(w, block, ue8m0)
    return ref.blockwise_cast_to_fp8(w, block, ue8m0)


def blockwise_dequant_fp8(q, scale_inv, block=128, dtype=None):
    import torch

    dtype = dtype or torch.bfloat16
    if _use_cuda(q):
        return _cuda().blockwise_dequant_fp8(q, scale_inv, block, dtype)
    return ref.blockwise_dequant_fp8(q, scale_inv, block, dtype)


def kv_cache_write(k, v, k_cache, v_cache, slots):
    """Scatter new K/V rows ``[T, Hkv, D]`` into a paged cache ``[blocks, block_size, Hkv, D]``
    at flat slot indices ``slots[T]`` (``block * block_size + offset``)."""
    if _use_cuda(k):
        return _cuda().kv_scatter(k, v, k_cache, v_cache, slots)
    kc = k_cache.view(-1, k.shape[1], k.shape[2])
    vc = v_cache.view(-1, v.shape[1], v.shape[2])
    kc[slots] = k
    vc[slots] = v


def qkv_post(qkv, nq, nkv, q_norm_w, k_norm_w, cos, sin, eps, k_cache=None, v_cache=None, slots=None, dense_kv=True):
    """Inference-side glue after the fused QKV projection: optional per-head RMSNorm of q and k, rotary
    embedding, and the write of the new K/V rows into the paged cache.  One kernel on CUDA (bf16,
    head_dim 128); the statement below elsewhere.  Returns ``(q, k, v)`` with ``k``/``v`` None when
    ``dense_kv`` is False (decode: attention reads the cache)."""
    hd = qkv.shape[1] // (nq + 2 * nkv)
    if (_use_cuda(qkv) and hd == 128 and qkv.dtype == torch.bfloat16 and not torch.is_grad_enabled()
            and cos.shape[-1] == 64):
        return _cuda().qkv_post(qkv, nq, nkv, q_norm_w, k_norm_w, cos, sin, eps, k_cache, v_cache, slots, dense_kv)
    T = qkv.shape[0]
    q = qkv[:, : nq * hd].reshape(T, nq, hd)
    k = qkv[:, nq * hd:(nq + nkv) * hd].reshape(T, nkv, hd)
    v = qkv[:, (nq + nkv) * hd:].reshape(T, nkv, hd)
    if q_norm_w is not None:
        q, k = rmsnorm(q, q_norm_w, eps), rmsnorm(k, k_norm_w, eps)
    rot = 2 * cos.shape[-1]
    if rot < hd:      # partial rotary (GLM-4, Qwen3.5): only the first ``rot`` dims of every head turn
        q = torch.cat([apply_rope(q[..., :rot].contiguous(), cos, sin), q[..., rot:]], -1)
        k = torch.cat([apply_rope(k[..., :rot].contiguous(), cos, sin), k[..., rot:]], -1)
    else:
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    if slots is not None:
        kv_cache_write(k, v, k_cache, v_cache, slots)
    return (q, k, v.contiguous()) if dense_kv else (q, None, None)


def linear_swiglu(x, w):
    """``swiglu(x @ w.T)`` with ``w`` = [gate; up]; fused split-K reduction + activation for decode shapes."""
    if _use_cuda(x) and x.shape[0] <= 256 and not torch.is_grad_enabled() and x.dim() == 2:
        return _cuda().linear_swiglu_skinny(x, w)
    return swiglu(linear(x, w))


def fp8_linear(x, w_q, w_scale_inv, block: int = 128):
    """``x @ dequant(w_q, w_scale_inv)^T`` with block-scaled e4m3 operands (weights: one scale per ``block x block``
    tile; activations quantised per row and ``block`` columns on the fly).  tcgen05 ``kind::f8f6f4`` on CUDA;
    elsewhere the dequantised product."""
    if _use_cuda(x) and block == 128:
        return _cuda().fp8_linear(x, w_q, w_scale_inv)
    w = blockwise_dequant_fp8(w_q, w_scale_inv, block, torch.float32)
    return (x.float() @ w.float().t()).to(torch.bfloat16)


def dgrad(dy, w):
    """dy[M,N] @ w[N,K] (input gradient of ``linear``)."""
    if _use_cuda(dy):
        return _cuda().matmul_nn(dy.contiguous(), w)
    return dy @ w


def wgrad(dy, x, w=None):
    """dy[M,N]^T @ x[M,K] (weight gradient of ``linear``).  When ``w`` carries an fp32
    ``main_grad`` buffer the CUDA path accumulates into it and returns ``None``."""
    if _use_cuda(dy):
        c = _cuda()
        mg = getattr(w, "main_grad", None) if w is not None else None
        import torch

        if mg is not None and mg.dtype == torch.float32 and mg.shape == w.shape:
            c.matmul_tn(dy.contiguous(), x.contiguous(), out=mg, accumulate=True)
            return None
        return c.matmul_tn(dy.contiguous(), x.contiguous())
    return dy.t() @ x
