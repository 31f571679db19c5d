"""Autograd wrappers around the in-tree sm_100a extension (``relax_b200/_C.so``).

Importing this module on a machine with a GPU but without the built extension
raises: CUDA tensors never fall back to library kernels silently.
"""
from __future__ import annotations

import importlib.util
import math
import os
from typing import Optional

import torch

_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C.so")
_C = None
_ERR: dict = {}
_MN_OK: Optional[bool] = None


def _load():
    global _C
    if _C is not None:
        return _C
    if not os.path.exists(_SO):
        raise RuntimeError(f"{_SO} is missing: build it with `python __graft_entry__.py` (nvcc, sm_100a)")
    spec = importlib.util.spec_from_file_location("relax_b200._C", _SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if os.environ.get("RELAX_B200_CRASH_TRACE", "0") == "1":
        mod.install_crash_handler()
    _C = mod
    return mod


def available() -> bool:
    if not torch.cuda.is_available():
        return False
    _load()
    return True


def err_flag(device=None) -> torch.Tensor:
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    if dev.type != "cuda":
        dev = torch.device("cuda", torch.cuda.current_device())
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _ERR:
        _ERR[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
    return _ERR[idx]


def check_error_flag(device=None):
    """Raise if any kernel recorded an error status (e.g. a bounded wait that ran out)."""
    f = err_flag(device)
    v = int(f.item())
    if v != 0:
        f.zero_()
        raise RuntimeError(f"sm_100a kernel reported error status {v} (1 = barrier wait timed out, 3 = peer wait timed out)")


# --------------------------------------------------------------------------- GEMM


_PAIR = os.environ.get("RELAX_B200_GEMM_PAIR", "1") == "1"


def gemm_raw(a, b, out, M, N, K, lda, ldb, ldc, a_mn=False, b_mn=False, accumulate=False, bias=None, force_bn=0,
             lbo_a=0, sbo_a=0, lbo_b=0, sbo_b=0, pair=None):
    """One GEMM launch.  Problems with at least one full 256-row pair tile go to the CTA-pair kernel
    (csrc/gemm2_sm100.cu: ``cta_group::2``, TMA-store / TMA-reduce epilogue); the rest, and anything with a bias,
    a forced tile width or a non-default descriptor, to the single-CTA kernel (csrc/gemm_sm100.cu)."""
    L = _load()
    use_pair = _PAIR if pair is None else pair
    if (use_pair and bias is None and force_bn == 0 and M >= 256 and N >= 128 and a.dtype == torch.bfloat16
            and not (lbo_a or sbo_a or lbo_b or sbo_b) and (out.dtype == torch.float32 or not accumulate)):
        if L.gemm_pair(a, b, out, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate, 256 if N >= 256 else 128,
                       err_flag(a.device)):
            return out
    L.gemm(a, b, out, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate, force_bn, lbo_a, sbo_a, lbo_b, sbo_b,
           err_flag(a.device))
    return out


def _rowmajor_2d(t):
    """Return (tensor, ld) such that the tensor is a row-major matrix with 16-byte aligned pitch."""
    if t.stride(-1) != 1 or t.stride(0) % 8 or t.stride(0) < t.shape[1] or t.data_ptr() % 16:
        t = t.contiguous()
        if t.shape[1] % 8:
            raise ValueError(f"GEMM operand inner dimension {t.shape[1]} must be a multiple of 8")
    return t, t.stride(0)


def mn_major_ok() -> bool:
    """One-time numerical self-check of the MN-major (transposed operand) tensor-core path
    against the K-major path on explicitly transposed copies."""
    global _MN_OK
    if _MN_OK is None:
        if os.environ.get("RELAX_B200_DISABLE_MN_MAJOR", "0") == "1":
            _MN_OK = False
            return False
        g = torch.Generator(device="cuda").manual_seed(1)
        M, N, K = 256, 192, 320
        at = torch.randn(K, M, device="cuda", generator=g).bfloat16()   # A stored transposed
        bt = torch.randn(K, N, device="cuda", generator=g).bfloat16()
        ref = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        gemm_raw(at.t().contiguous(), bt.t().contiguous(), ref, M, N, K, K, K, N)
        out = torch.empty_like(ref)
        gemm_raw(at, bt, out, M, N, K, M, N, N, a_mn=True, b_mn=True)
        _MN_OK = bool(torch.allclose(out.float(), ref.float(), atol=1e-2, rtol=1e-2))
    return _MN_OK


def matmul_nt(x, w, bias=None, out_dtype=None, out=None, accumulate=False):
    """x[M,K] @ w[N,K]^T."""
    x, lda = _rowmajor_2d(x)
    w, ldb = _rowmajor_2d(w)
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or x.dtype, device=x.device)
    return gemm_raw(x, w, out, M, N, K, lda, ldb, out.stride(0), bias=bias, accumulate=accumulate)


def matmul_nn(a, b, out=None, out_dtype=None):
    """a[M,K] @ b[K,N]  (b row-major: the MN-major B operand)."""
    a, lda = _rowmajor_2d(a)
    M, K = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    if mn_major_ok() and N % 8 == 0:
        b, ldb = _rowmajor_2d(b)
        return gemm_raw(a, b, out, M, N, K, lda, ldb, out.stride(0), b_mn=True)
    bt = b.t().contiguous()
    return gemm_raw(a, bt, out, M, N, K, lda, bt.stride(0), out.stride(0))


def matmul_tn(a, b, out=None, out_dtype=None, accumulate=False):
    """a[K,M]^T @ b[K,N] -> [M,N]  (both operands MN-major: weight gradients)."""
    K, M = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    if mn_major_ok() and M % 8 == 0 and N % 8 == 0:
        a, lda = _rowmajor_2d(a)
        b, ldb = _rowmajor_2d(b)
        return gemm_raw(a, b, out, M, N, K, lda, ldb, out.stride(0), a_mn=True, b_mn=True, accumulate=accumulate)
    at, bt = a.t().contiguous(), b.t().contiguous()
    return gemm_raw(at, bt, out, M, N, K, at.stride(0), bt.stride(0), out.stride(0), accumulate=accumulate)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        return matmul_nt(x, w, bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = matmul_nn(dy, w) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None and mg.dtype == torch.float32 and mg.shape == w.shape and mg.stride(-1) == 1:
                # weight-gradient GEMM accumulates straight into the fp32 gradient buffer of the
                # distributed optimizer: no temporary, no separate add pass
                matmul_tn(dy, x, out=mg, accumulate=True)
            else:
                dw = matmul_tn(dy, x)
        db = dy.sum(0) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db


def linear(x, w, bias=None):
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if x2.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("the sm_100a GEMM takes bf16/fp16 inputs")
    if w.dim() != 2:
        raise ValueError("weight must be 2-D")
    if x2.shape[0] <= 256 and not (torch.is_grad_enabled() and (x2.requires_grad or w.requires_grad)) \
            and w.is_contiguous() and w.shape[0] % 64 == 0:
        y = matmul_nt_skinny(x2, w, bias)
        bias = None
    elif not w.is_contiguous() and w.t().is_contiguous():
        # y = x @ (w^T stored row-major)  ->  NN product
        y = _LinearNN.apply(x2, w.t())
    else:
        y = _Linear.apply(x2, w, bias)
        bias = None
    if bias is not None:
        y = y + bias
    return y.reshape(*shp[:-1], y.shape[-1])


_DECODE_GEMM = os.environ.get("RELAX_B200_DECODE_GEMM", "1") == "1"


def _decode_gemm(x, w, swiglu: bool):
    """Weight-streaming decode GEMM (csrc/gemm_decode_sm100.cu) when the shape is in its range, else None."""
    if not _DECODE_GEMM or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.shape[0] > 128:
        return None     # above 128 rows the 2-stage ring of the 256-column variant loses to the other paths (measured)
    if w.stride(1) != 1 or w.stride(0) % 8 or w.data_ptr() % 16:
        return None
    N = w.shape[0]
    out = torch.empty(x.shape[0], N // 2 if swiglu else N, dtype=x.dtype, device=x.device)
    if _load().decode_gemm(x, w, out, swiglu, 0, err_flag(x.device)):
        return out
    return None


def _wide_pair_gemm(x, w):
    """129..256 token rows against a wide weight (N >= 6144: at least 24 pair tiles of 256 x 256): one row of CTA-pair
    tiles of the training GEMM beats split-K here (measured on B200 at 160 and 256 rows: 33 vs 52 us at N = 12288,
    31 vs 50 us at N = 6144; below that split-K wins).  Returns None when the shape is outside that range."""
    M, K = x.shape
    N = w.shape[0]
    if not (_PAIR and 128 < M <= 256 and N >= 6144 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.is_contiguous()):
        return None
    out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    if _load().gemm_pair(x, w, out, M, N, K, x.stride(0), w.stride(0), N, False, False, False, 256, err_flag(x.device)):
        return out
    return None


def matmul_nt_skinny(x, w, bias=None, residual=None):
    """x[M, K] @ w[N, K]^T for decode (a few hundred rows at most): when the N tiles alone cannot fill the SMs the
    reduction dimension is split across CTAs (fp32 partials in a workspace, one small reduce
    kernel that also adds bias / residual)."""
    x, _ = _rowmajor_2d(x)
    M, K = x.shape
    N = w.shape[0]
    C = _load()
    if bias is None and residual is None:
        y = _decode_gemm(x, w, False)
        if y is None:
            y = _wide_pair_gemm(x, w)
        if y is not None:
            return y
    splits, bn = C.gemm_splitk_plan(M, N, K)
    out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    if splits <= 1:
        gemm_raw(x, w, out, M, N, K, x.stride(0), w.stride(0), N, bias=bias)
        return out if residual is None else out + residual
    ws = torch.empty(splits * M * N, dtype=torch.float32, device=x.device)
    C.gemm_splitk(x, w, out, bias, residual, ws, splits, bn, err_flag(x.device))
    return out


def linear_swiglu_skinny(x, w):
    """``swiglu(x @ w.T)`` for decode (``w`` = [gate; up] rows): split-K partial sums, then ONE kernel that
    reduces them and applies the activation, instead of reduce + swiglu."""
    x, _ = _rowmajor_2d(x)
    M, K = x.shape
    N = w.shape[0]
    C = _load()
    y = _decode_gemm(x, w, True)
    if y is not None:
        return y
    y = _wide_pair_gemm(x, w)
    if y is not None:
        return swiglu(y)
    splits, bn = C.gemm_splitk_plan(M, N, K)
    if splits <= 1 or x.dtype != torch.bfloat16 or (N // 2) % 4:
        return swiglu(linear(x, w))
    ws = torch.empty(splits * M * N, dtype=torch.float32, device=x.device)
    C.gemm_splitk_partial(x, w, ws, splits, bn, err_flag(x.device))
    out = torch.empty(M, N // 2, dtype=x.dtype, device=x.device)
    C.splitk_swiglu(ws, out, splits)
    return out


def qkv_post(qkv, nq, nkv, q_norm_w, k_norm_w, cos, sin, eps, k_cache=None, v_cache=None, slots=None, dense_kv=True):
    """Per-head q/k RMSNorm (optional) + rotary embedding + KV-cache write in one launch.
    Returns ``(q, k, v)`` as ``[T, heads, 128]``; ``k``/``v`` are None unless ``dense_kv``."""
    T = qkv.shape[0]
    q = torch.empty(T, nq, 128, dtype=qkv.dtype, device=qkv.device)
    k = torch.empty(T, nkv, 128, dtype=qkv.dtype, device=qkv.device) if dense_kv else None
    v = torch.empty(T, nkv, 128, dtype=qkv.dtype, device=qkv.device) if dense_kv else None
    _load().qkv_post(qkv, q_norm_w, k_norm_w, cos.contiguous(), sin.contiguous(), q, k, v, k_cache, v_cache, slots, nq, nkv,
                     float(eps))
    return q, k, v


def quantize_rows_fp8(x, block: int = 128):
    """Per-row, per-``block`` columns e4m3 quantisation of activations: ``(q [M, K] float8_e4m3fn, scale [M, K/block])``
    with ``x ~ q * scale``."""
    M, K = x.shape
    kb = (K + block - 1) // block
    xp = torch.nn.functional.pad(x.float(), (0, kb * block - K)).view(M, kb, block)
    scale = xp.abs().amax(-1).clamp_min(1e-12) / 448.0
    q = (xp / scale.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(M, kb * block)[:, :K].contiguous()
    return q, scale.contiguous()


def fp8_linear(x, w_q, w_scale_inv, x_q=None, x_scale=None):
    """``x @ dequant(w_q)^T`` on the fp8 tensor cores with block scaling: weights are e4m3 with one scale per
    128 x 128 block (``weight_scale_inv`` of :func:`blockwise_cast_to_fp8`), activations are quantised per row and
    128 columns here unless given.  Output bf16."""
    x2 = x.reshape(-1, x.shape[-1])
    if x_q is None:
        x_q, x_scale = quantize_rows_fp8(x2)
    out = torch.empty(x2.shape[0], w_q.shape[0], dtype=torch.bfloat16, device=x.device)
    _load().gemm_fp8(x_q, x_scale.float().contiguous(), w_q, w_scale_inv.float().contiguous(), out, err_flag(x.device))
    return out.reshape(*x.shape[:-1], w_q.shape[0])


class _LinearNN(torch.autograd.Function):
    """y = x @ b with b[K,N] row-major (used when the caller passes ``w.t()``)."""

    @staticmethod
    def forward(ctx, x, b):
        ctx.save_for_backward(x, b)
        return matmul_nn(x, b)

    @staticmethod
    def backward(ctx, dy):
        x, b = ctx.saved_tensors
        dy = dy.contiguous()
        dx = matmul_nt(dy, b) if ctx.needs_input_grad[0] else None
        db = matmul_tn(x, dy) if ctx.needs_input_grad[1] else None
        return dx, db


# --------------------------------------------------------------------------- norms / elementwise


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        x = x.contiguous()
        cols = x.shape[-1]
        rows = x.numel() // cols
        y = torch.empty_like(x)
        _load().rmsnorm_fwd(x, None, w, y, None, rows, cols, eps)
        ctx.save_for_backward(x, w)
        ctx.eps = eps
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        cols = x.shape[-1]
        rows = x.numel() // cols
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.empty_like(w)
        C = _load()
        scratch = torch.empty(C.rmsnorm_bwd_parts(rows, cols) * cols, dtype=torch.float32, device=x.device)
        C.rmsnorm_bwd(x, w, dy, dx, dw, scratch, rows, cols, ctx.eps)
        return dx, dw, None


def rmsnorm(x, w, eps=1e-6):
    return _RMSNorm.apply(x, w, eps)


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, w, eps):
        x, res = x.contiguous(), res.contiguous()
        cols = x.shape[-1]
        rows = x.numel() // cols
        y, r = torch.empty_like(x), torch.empty_like(x)
        _load().rmsnorm_fwd(x, res, w, y, r, rows, cols, eps)
        ctx.save_for_backward(r, w)
        ctx.eps = eps
        return y, r

    @staticmethod
    def backward(ctx, dy, dr):
        r, w = ctx.saved_tensors
        cols = r.shape[-1]
        rows = r.numel() // cols
        dx = torch.empty_like(r)
        dw = torch.empty_like(w)
        C = _load()
        scratch = torch.empty(C.rmsnorm_bwd_parts(rows, cols) * cols, dtype=torch.float32, device=r.device)
        C.rmsnorm_bwd(r, w, dy.contiguous(), dx, dw, scratch, rows, cols, ctx.eps)
        if dr is not None:
            dx = dx + dr
        return dx, dx, dw, None


def add_rmsnorm(x, res, w, eps=1e-6):
    return _AddRMSNorm.apply(x, res, w, eps)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        x = x.contiguous()
        T, H, D = x.shape
        y = torch.empty_like(x)
        cos, sin = cos.contiguous(), sin.contiguous()
        _load().rope(x, y, cos, sin, T, H, D, False)
        ctx.save_for_backward(cos, sin)
        return y

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        dy = dy.contiguous()
        T, H, D = dy.shape
        dx = torch.empty_like(dy)
        _load().rope(dy, dx, cos, sin, T, H, D, True)
        return dx, None, None


def apply_rope(x, cos, sin):
    return _Rope.apply(x, cos.float(), sin.float())


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        gu = gu.contiguous()
        F = gu.shape[-1] // 2
        rows = gu.numel() // (2 * F)
        out = torch.empty(*gu.shape[:-1], F, dtype=gu.dtype, device=gu.device)
        _load().swiglu_fwd(gu, out, rows, F)
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        F = gu.shape[-1] // 2
        rows = gu.numel() // (2 * F)
        din = torch.empty_like(gu)
        _load().swiglu_bwd(gu, dout.contiguous(), din, rows, F)
        return din


def swiglu(gate_up):
    return _SwiGLU.apply(gate_up)


# --------------------------------------------------------------------------- optimizer / misc


def fused_adam(pshard, master, gshard, exp_avg, exp_avg_sq, step, lr, b1, b2, eps, wd, gscale, split):
    _load().adam(pshard, master, gshard, exp_avg, exp_avg_sq, step, lr, b1, b2, eps, wd, gscale, split)


def sumsq(x) -> torch.Tensor:
    out = torch.zeros(1, dtype=torch.float32, device=x.device)
    _load().sumsq(x.contiguous().view(-1), out)
    return out


def kv_scatter(k, v, k_cache, v_cache, slots):
    """k/v ``[T, H, D]`` (possibly strided views of a fused qkv buffer) -> cache rows ``slots[T]``."""
    T = k.shape[0]
    row = k.shape[1] * k.shape[2]
    if k.stride(2) != 1 or k.stride(1) != k.shape[2]:
        k = k.contiguous()
    if v.stride(2) != 1 or v.stride(1) != v.shape[2]:
        v = v.contiguous()
    _load().kv_scatter(k, v, k_cache, v_cache, slots, T, row, k.stride(0), v.stride(0))


def fake_int4_quant(x, block_m, block_n, sym=True):
    x = x.contiguous()
    M, N = x.shape
    gm, gn = (M + block_m - 1) // block_m, (N + block_n - 1) // block_n
    out = torch.empty_like(x)
    scale = torch.empty(gm, gn, dtype=x.dtype, device=x.device)
    zero = torch.empty(gm, gn, dtype=x.dtype, device=x.device)
    _load().int4_fake_quant(x, out, scale, zero, block_m, block_n, sym)
    return out, scale, zero


def blockwise_cast_to_fp8(w, block=128, ue8m0=False):
    w = w.contiguous()
    M, N = w.shape
    q = torch.empty(M, N, dtype=torch.float8_e4m3fn, device=w.device)
    scale = torch.empty((M + block - 1) // block, (N + block - 1) // block, dtype=torch.float32, device=w.device)
    _load().fp8_block_cast(w, q, scale, block, ue8m0)
    return q, scale


def blockwise_dequant_fp8(q, scale_inv, block=128, dtype=torch.bfloat16):
    out = torch.empty(q.shape, dtype=dtype, device=q.device)
    _load().fp8_block_dequant(q.contiguous(), scale_inv.contiguous(), out, block)
    return out


# --------------------------------------------------------------------------- weight-sync copy table


class CopyTable:
    def __init__(self, table, chunk_start, n_desc, total_chunks, chunk_rows, elem_size, keepalive):
        self.table, self.chunk_start = table, chunk_start
        self.n_desc, self.total_chunks, self.chunk_rows, self.elem_size = n_desc, total_chunks, chunk_rows, elem_size
        self.keepalive = keepalive


def build_copy_table_raw(entries, device, elem_size: int, chunk_bytes: int = 1 << 18) -> CopyTable:
    """entries: (src_ptr, dst_ptr, rows, cols, src_ld, dst_ld) in elements.  Large blocks are
    split into chunks of about ``chunk_bytes`` so the copy spreads over all SMs."""
    import struct

    raw = bytearray()
    starts, total = [], 0
    chunk_rows_list = []
    # one global chunk_rows keeps the kernel simple: rows per chunk chosen from the widest block
    max_cols = max((e[3] for e in entries), default=1)
    chunk_rows = max(1, chunk_bytes // max(1, max_cols * elem_size))
    for (s, d, rows, cols, sld, dld) in entries:
        raw += struct.pack("<QQiiii", s, d, rows, cols, sld, dld)
        starts.append(total)
        total += (rows + chunk_rows - 1) // chunk_rows
    table = torch.frombuffer(raw, dtype=torch.uint8).to(device)
    cs = torch.tensor(starts, dtype=torch.int32, device=device)
    return CopyTable(table, cs, len(entries), total, chunk_rows, elem_size, None)


def copy_entries(blocks, trainer_params: dict, dst_params: dict) -> list:
    """Raw ``(src_ptr, dst_ptr, rows, cols, src_ld, dst_ld)`` entries of plan blocks; ``dst_params`` maps rollout
    parameter names to tensors, which may be views of ANOTHER GPU's memory mapped into this process."""
    entries = []
    es = next(iter(trainer_params.values())).element_size()
    for b in blocks:
        src = trainer_params[b.src_name]
        dst = dst_params[b.dst_name]
        s2 = src[b.src_batch] if src.dim() == 3 else (src.view(1, -1) if src.dim() == 1 else src)
        d2 = dst[b.dst_batch] if dst.dim() == 3 else (dst.view(1, -1) if dst.dim() == 1 else dst)
        sp = s2.data_ptr() + (b.src_row * s2.stride(0) + b.src_col) * es
        dp = d2.data_ptr() + (b.dst_row * d2.stride(0) + b.dst_col) * es
        entries.append((sp, dp, b.rows, b.cols, s2.stride(0), d2.stride(0)))
    return entries


def build_copy_table(blocks, trainer_params: dict, rollout_weights) -> CopyTable:
    es = next(iter(trainer_params.values())).element_size()
    t = build_copy_table_raw(copy_entries(blocks, trainer_params, rollout_weights.p), rollout_weights.device, es)
    t.keepalive = (trainer_params, rollout_weights)
    return t


def run_copy_table(t: CopyTable):
    _load().copy_table(t.table, t.n_desc, t.chunk_start, t.total_chunks, t.chunk_rows, t.elem_size)


# --------------------------------------------------------------------------- flash attention (training / prefill)


def _tok_head_view(t):
    """[T, H, 128] with unit inner stride and 16-byte aligned outer strides, else a contiguous copy."""
    if t.stride(2) != 1 or t.stride(0) % 8 or t.stride(1) % 8 or t.data_ptr() % 16:
        t = t.contiguous()
    return t


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, causal, scale, max_q_blocks, max_kv_blocks):
        q, k, v = _tok_head_view(q), _tok_head_view(k), _tok_head_view(v)
        Tq, Hq, D = q.shape
        o = torch.empty(Tq, Hq, D, dtype=q.dtype, device=q.device)
        lse = torch.empty(Hq, Tq, dtype=torch.float32, device=q.device)
        _load().fa_fwd(q, k, v, o, lse, cu_q, cu_k, max_q_blocks, causal, scale, err_flag(q.device))
        ctx.save_for_backward(q, k, v, o, lse, cu_q, cu_k)
        ctx.causal, ctx.scale, ctx.max_kv_blocks = causal, scale, max_kv_blocks
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, cu_q, cu_k = ctx.saved_tensors
        q, k, v, do = q.contiguous(), k.contiguous(), v.contiguous(), do.contiguous()
        Tq, Hq, D = q.shape
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty(Hq, Tq, dtype=torch.float32, device=q.device)
        dq_acc = torch.empty(Tq, Hq, D, dtype=torch.float32, device=q.device)
        _load().fa_bwd(q, k, v, o, do, lse, dq, dk, dv, delta, dq_acc, cu_q, cu_k, ctx.max_kv_blocks, ctx.causal,
                       ctx.scale, err_flag(q.device))
        return dq, dk, dv, None, None, None, None, None, None


def attention_varlen(q, k, v, cu_seqlens, causal=True, scale=None, cu_seqlens_k=None, max_seqlen=None):
    """Packed varlen attention; q [Tq, Hq, 128], k/v [Tk, Hkv, 128] bf16."""
    if q.dtype != torch.bfloat16 or q.shape[-1] != 128:
        raise NotImplementedError("the sm_100a attention kernel handles bf16 with head_dim 128")
    cu_q = cu_seqlens.to(torch.int32)
    cu_k = cu_q if cu_seqlens_k is None else cu_seqlens_k.to(torch.int32)
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    nseq = cu_q.numel() - 1
    # upper bounds of the tile counts (no host sync): every sequence adds at most one partial tile
    max_q_blocks = (q.shape[0] + 127) // 128 + nseq
    max_kv_blocks = (k.shape[0] + 127) // 128 + nseq
    return _FlashAttn.apply(q, k, v, cu_q, cu_k, bool(causal), float(scale), max_q_blocks, max_kv_blocks)


# --------------------------------------------------------------------------- rollout kernels


def paged_decode_attention(q, k_cache, v_cache, block_tables, context_lens, scale=None, max_ctx=None, splits=None,
                           version=None):
    B, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if max_ctx is None:
        max_ctx = block_tables.shape[1] * k_cache.shape[1]
    C = _load()
    if splits is None:
        splits = int(os.environ.get("RELAX_B200_DECODE_SPLITS", "0")) or C.decode_attn_splits(B, Hkv, max_ctx)
        if B * Hkv >= 148:
            splits = 1   # enough CTAs already; splitting only adds the combine pass
    if version is None:
        version = int(os.environ.get("RELAX_B200_DECODE_ATTN_VERSION", "3"))
    if version == 3 and k_cache.shape[1] != 16:
        version = 1   # the tensor-core kernel gathers 16-token pages
    out = torch.empty_like(q)
    po = pm = None
    if splits > 1:
        po = torch.empty(B * Hq * splits * D, dtype=torch.float32, device=q.device)
        pm = torch.empty(B * Hq * splits * 2, dtype=torch.float32, device=q.device)
    C.decode_attn(q.contiguous(), k_cache, v_cache, block_tables.to(torch.int32).contiguous(),
                  context_lens.to(torch.int32).contiguous(), out, po, pm, max_ctx, scale, splits, version,
                  err_flag(q.device))
    return out


def sample(logits, temperature, top_k, top_p, uniform):
    """Rows of bf16 or fp32 logits (unit inner stride; any row pitch) -> ``(token int64 [B], log-prob fp32 [B])``."""
    if logits.dtype not in (torch.bfloat16, torch.float32):
        logits = logits.float()
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    B, V = logits.shape
    tok = torch.empty(B, dtype=torch.int64, device=logits.device)
    lp = torch.empty(B, dtype=torch.float32, device=logits.device)
    _load().sample_v2(logits, temperature.float().contiguous(), top_k.to(torch.int64).contiguous(),
                      top_p.float().contiguous(), uniform.float().contiguous(), tok, lp, V)
    return tok, lp


def decode_advance(tok_new, lp_new, st, block_size: int):
    """Device-side tail of one decode step (see :func:`relax_b200.ops.reference.decode_advance` for the statement)."""
    _load().decode_advance(tok_new, lp_new, st["tok"], st["pos"], st["ctx"], st["slots"], st["bt"], int(block_size),
                           st["active"], st["remain"], st["eos"], st["stop"], st["out_tok"], st["out_lp"], st["counter"],
                           st["u_all"], st["u"])


class _TopKRouter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, norm):
        logits = logits.float().contiguous()
        T, E = logits.shape
        w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
        idx = torch.empty(T, k, dtype=torch.int64, device=logits.device)
        probs = torch.empty(T, E, dtype=torch.float32, device=logits.device)
        _load().topk_router(logits, k, norm, w, idx, probs)
        ctx.save_for_backward(probs, idx, w)
        ctx.norm = norm
        ctx.mark_non_differentiable(idx)
        return w, idx, probs

    @staticmethod
    def backward(ctx, dw, _didx, dprobs):
        probs, idx, w = ctx.saved_tensors
        # gradient w.r.t. probs from the (optionally renormalised) selected weights
        gp = torch.zeros_like(probs) if dprobs is None else dprobs.clone()
        if dw is not None:
            if ctx.norm:
                sel = probs.gather(-1, idx)
                ssum = sel.sum(-1, keepdim=True)
                dsel = (dw - (dw * w).sum(-1, keepdim=True)) / ssum
            else:
                dsel = dw
            gp.scatter_add_(-1, idx, dsel)
        # softmax backward
        dlogits = probs * (gp - (gp * probs).sum(-1, keepdim=True))
        return dlogits, None, None


def topk_router(logits, top_k, norm_topk_prob=True):
    return _TopKRouter.apply(logits, int(top_k), bool(norm_topk_prob))


# --------------------------------------------------------------------------- fused LM head + log-prob / entropy


class _FusedLMHead(torch.autograd.Function):
    CHUNK = 4096
    _dlogits: dict = {}       # (device, dtype) -> flat scratch for the chunk's d(logits), reused by every backward

    @staticmethod
    def forward(ctx, hidden, weight, targets, tp_group, vocab_start, with_entropy, temperature):
        import torch.distributed as dist

        C = _load()
        h = hidden if (hidden.stride(1) == 1 and hidden.stride(0) % 8 == 0) else hidden.contiguous()
        w = weight if (weight.stride(1) == 1 and weight.stride(0) % 8 == 0) else weight.contiguous()
        T, V = h.shape[0], w.shape[0]
        inv_t = 1.0 / float(temperature)
        tp = tp_group is not None and dist.is_initialized() and dist.get_world_size(tp_group) > 1
        if T == 0:
            z = torch.zeros(0, dtype=torch.float32, device=h.device)
            ctx.save_for_backward(h, w, targets, z, z)
            ctx.meta = (tp_group, vocab_start, inv_t, with_entropy, weight)
            return z, z.clone()
        splits = C.lm_head_splits(T, V)
        part = torch.empty(T, splits, 4, dtype=torch.float32, device=h.device)
        C.lm_head_logprob(h, w, targets.contiguous(), part, vocab_start, inv_t, splits, err_flag(h.device))
        m = part[..., 0]
        gm = m.max(1).values
        if tp:
            dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=tp_group)
        sc = torch.exp(m - gm[:, None])
        zt = part[..., 3].max(1).values
        found = torch.isfinite(zt)
        acc = torch.stack([(part[..., 1] * sc).sum(1), (part[..., 2] * sc).sum(1), torch.where(found, zt, torch.zeros_like(zt))])
        if tp:
            dist.all_reduce(acc, group=tp_group)
        s, u, zt = acc[0], acc[1], acc[2]
        logz = gm + torch.log(s)
        ez = u / s
        lp = zt - logz
        ent = logz - ez if with_entropy else torch.zeros_like(lp)
        ctx.save_for_backward(h, w, targets, logz, ez)
        ctx.meta = (tp_group, vocab_start, inv_t, with_entropy, weight)
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        h, w, targets, logz, ez = ctx.saved_tensors
        tp_group, vocab_start, inv_t, with_entropy, weight = ctx.meta
        C = _load()
        T, H = h.shape
        V = w.shape[0]
        dh = torch.empty_like(h)
        main_grad = getattr(weight, "main_grad", None)
        direct = main_grad is not None and main_grad.dtype == torch.float32 and main_grad.shape == weight.shape \
            and w.data_ptr() == weight.data_ptr()
        dw32 = main_grad if direct else torch.zeros(V, H, dtype=torch.float32, device=h.device)
        if main_grad is not None and not direct and main_grad.dtype == torch.float32 and w.shape[0] < weight.shape[0] \
                and w.data_ptr() == weight.data_ptr():
            dw32, direct = main_grad[:V], True   # vocabulary padding rows sliced off by the caller
        stats = torch.stack([logz, ez], 1).contiguous()
        g_lp = (g_lp if g_lp is not None else torch.zeros_like(logz)).float().contiguous()
        g_en = g_ent.float().contiguous() if (with_entropy and g_ent is not None) else None
        tg = targets.contiguous()
        ck = _FusedLMHead.CHUNK
        # d(logits) of one chunk: up to 4096 x V (1.2 GB at V = 152k).  Kept across calls: a fresh allocation of that
        # size per micro-batch does not fit the blocks the caching allocator has left and costs a cudaMalloc every
        # time (about 12 ms during which the device runs dry - measured)
        key = (h.device, h.dtype)
        buf = _FusedLMHead._dlogits.get(key)
        need = min(ck, T) * V
        if buf is None or buf.numel() < need:
            buf = None
            _FusedLMHead._dlogits.pop(key, None)
            buf = _FusedLMHead._dlogits[key] = torch.empty(need, dtype=h.dtype, device=h.device)
        buf = buf[:need].view(min(ck, T), V)
        for s in range(0, T, ck):
            e = min(T, s + ck)
            d = buf[: e - s]
            C.lm_head_dlogits(h[s:e], w, tg[s:e], stats[s:e], g_lp[s:e], None if g_en is None else g_en[s:e], d,
                              vocab_start, inv_t, err_flag(h.device))
            matmul_nn(d, w, out=dh[s:e])
            matmul_tn(d, h[s:e], out=dw32, accumulate=True)
        dw = None if direct else dw32.to(weight.dtype)
        if dw is not None and dw.shape != weight.shape:
            full = torch.zeros_like(weight)
            full[: dw.shape[0]] = dw
            dw = full
        return dh, dw, None, None, None, None, None


def fused_lm_head_logprob(hidden, weight, targets, tp_group=None, vocab_start=0, with_entropy=True, temperature=1.0):
    if hidden.dtype != torch.bfloat16:
        raise TypeError("fused LM head expects bf16 hidden states")
    return _FusedLMHead.apply(hidden, weight, targets, tp_group, vocab_start, with_entropy, temperature)


# --------------------------------------------------------------------------- fused policy loss


class _PolicyLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ppo_kl, adv, eps_clip, eps_clip_high, eps_clip_c):
        kl = ppo_kl.detach().float().contiguous()
        loss, clip, g = (torch.empty_like(kl) for _ in range(3))
        _load().policy_loss(kl, adv.detach().float().contiguous().expand_as(kl).contiguous(), loss, clip, g,
                            float(eps_clip), float(eps_clip_high), float(eps_clip_c or 0.0))
        ctx.save_for_backward(g)
        ctx.mark_non_differentiable(clip)
        return loss, clip

    @staticmethod
    def backward(ctx, dloss, _dclip):
        (g,) = ctx.saved_tensors
        return dloss * g, None, None, None, None


def policy_loss(ppo_kl, advantages, eps_clip, eps_clip_high, eps_clip_c=None):
    """``(loss, clipfrac)`` per token of the PPO clipped surrogate in one kernel; the same pass writes
    d loss / d ppo_kl, so backward is one multiply.  Advantages are treated as constants."""
    return _PolicyLoss.apply(ppo_kl, advantages, eps_clip, eps_clip_high, eps_clip_c)


# --------------------------------------------------------------------------- grouped (MoE expert) GEMM


class _GroupedLinear(torch.autograd.Function):
    """``y[row] = x[row] @ w[expert(row)].T`` over an expert-sorted, 128-row aligned token buffer: ONE kernel launch
    per product for all local experts, tile -> expert map read on the device (csrc/grouped_gemm_sm100.cu)."""

    @staticmethod
    def forward(ctx, x, w, tile_expert, expert_rows):
        x = x.contiguous()
        wc = w if w.is_contiguous() else w.contiguous()
        y = torch.empty(x.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
        _load().grouped_gemm_fwd(x, wc, y, tile_expert, err_flag(x.device))
        ctx.save_for_backward(x, wc, tile_expert, expert_rows)
        ctx.weight = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wc, tile_expert, expert_rows = ctx.saved_tensors
        w = ctx.weight
        dy = dy.contiguous()
        L = _load()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            L.grouped_gemm_dgrad(dy, wc, dx, tile_expert, err_flag(x.device))
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None and mg.dtype == torch.float32 and mg.shape == w.shape and mg.is_contiguous():
                L.grouped_gemm_wgrad(dy, x, mg, expert_rows, True, err_flag(x.device))
            else:
                dw = torch.empty_like(wc)
                L.grouped_gemm_wgrad(dy, x, dw, expert_rows, False, err_flag(x.device))
        return dx, dw, None, None


def grouped_linear(x, w, tile_expert, expert_rows):
    if x.dtype != torch.bfloat16 or x.shape[0] % 128 or w.shape[1] % 64 or w.shape[2] % 64:
        raise ValueError("grouped GEMM: bf16, token rows padded to 128 per expert, expert dims multiples of 64")
    return _GroupedLinear.apply(x, w, tile_expert, expert_rows)


def launch_count() -> int:
    """Number of kernels of this extension launched since the last reset (all threads)."""
    return int(_load().launch_count())


def reset_launch_count():
    _load().reset_launch_count()
