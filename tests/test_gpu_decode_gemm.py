"""Split-K GEMM for skinny (decode) problems against an fp32 reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(80, 4096, 12288), (1, 4096, 4096), (128, 6144, 4096), (37, 1024, 2048), (64, 24576, 4096),
                                   (256, 3072, 4096), (300, 4096, 6144)])
def test_skinny_linear_splitk(M, N, K):
    from relax_b200.ops import cuda as C

    assert C.available()
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    b = torch.randn(N, device="cuda", generator=g).bfloat16()
    r = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    ref = x.float() @ w.float().t()
    tol = 0.02 * math.sqrt(K) * 0.05 + 0.05
    with torch.no_grad():
        y = C.linear(x, w)
        assert (y.float() - ref).abs().max() < tol
        y2 = C.matmul_nt_skinny(x, w, b, r)
        assert (y2.float() - (ref + b.float() + r.float())).abs().max() < tol + 0.05
    splits, bn = C._load().gemm_splitk_plan(M, N, K)
    assert splits >= 1 and bn in (64, 128)
    C.check_error_flag()


@pytest.mark.gpu
@pytest.mark.parametrize("norm", [True, False])
@pytest.mark.parametrize("dense", [True, False])
def test_qkv_post_matches_separate_kernels(norm, dense):
    """Fused q/k norm + rope + cache write against the chain of separate operators."""
    from relax_b200 import ops
    from relax_b200.ops import reference as R

    dev = "cuda"
    torch.manual_seed(3)
    T, nq, nkv, hd, bs, nb = 37, 8, 2, 128, 16, 9
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, device=dev).bfloat16()
    qw = (1 + 0.1 * torch.randn(hd, device=dev)).bfloat16() if norm else None
    kw = (1 + 0.1 * torch.randn(hd, device=dev)).bfloat16() if norm else None
    pos = torch.randint(0, 4000, (T,), device=dev)
    cos, sin = R.rope_cos_sin(pos, hd, 1e6)
    slots = torch.randperm(nb * bs, device=dev)[:T].to(torch.int64)
    slots[5] = -1
    kc = torch.zeros(nb, bs, nkv, hd, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    with torch.no_grad():
        q, k, v = ops.qkv_post(qkv, nq, nkv, qw, kw, cos, sin, 1e-6, kc, vc, slots, dense)
    # reference: fp32 statement of the same chain with bf16 rounding between the stages
    qr = qkv[:, : nq * hd].reshape(T, nq, hd)
    kr = qkv[:, nq * hd:(nq + nkv) * hd].reshape(T, nkv, hd)
    vr = qkv[:, (nq + nkv) * hd:].reshape(T, nkv, hd)
    if norm:
        qr, kr = R.rmsnorm(qr, qw, 1e-6), R.rmsnorm(kr, kw, 1e-6)
    qr, kr = R.apply_rope(qr, cos, sin), R.apply_rope(kr, cos, sin)
    torch.testing.assert_close(q.float(), qr.float(), atol=2e-2, rtol=2e-2)
    if dense:
        torch.testing.assert_close(k.float(), kr.float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(v.float(), vr.float(), atol=0, rtol=0)
    else:
        assert k is None and v is None
    live = slots >= 0
    torch.testing.assert_close(kc.view(-1, nkv, hd)[slots[live]].float(), kr[live].float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(vc.view(-1, nkv, hd)[slots[live]].float(), vr[live].float(), atol=0, rtol=0)
    assert float(kc.view(-1, nkv, hd).abs().sum(-1).sum(-1).ne(0).sum()) == int(live.sum())


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 48, 128, 256])
def test_linear_swiglu_skinny(M):
    from relax_b200 import ops

    dev = "cuda"
    torch.manual_seed(5)
    K, F = 1024, 1536
    x = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(2 * F, K, device=dev) * 0.05).bfloat16()
    with torch.no_grad():
        y = ops.linear_swiglu(x, w)
    z = x.float() @ w.float().t()
    g, u = z[:, :F], z[:, F:]
    ref = torch.nn.functional.silu(g) * u
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(16, 1024, 512), (128, 4096, 4096), (100, 512, 12288)])
def test_single_rank_gemm_reduce_residual_rmsnorm(M, N, K):
    """With one rank the peer-reduce kernel is a split-K GEMM + reduction + residual + RMSNorm in one launch."""
    from relax_b200.ops import cuda as C
    from relax_b200.parallel.state import GroupInfo
    from relax_b200.parallel.symm_mem import SymmComm

    dev = torch.device("cuda", 0)
    torch.manual_seed(11)
    comm = SymmComm(GroupInfo(None, (0,), 0), dev, workspace_mb=64)
    for rep in range(3):
        x = torch.randn(M, K, device=dev).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.03).bfloat16()
        res = torch.randn(M, N, device=dev).bfloat16()
        nw = (1 + 0.1 * torch.randn(N, device=dev)).bfloat16()
        h, y = comm.gemm_ar_add_rmsnorm(x, w, res, nw, 1e-6)
        C.check_error_flag(dev)
        ref_h = (res.float() + x.float() @ w.float().t()).bfloat16().float()
        ref_y = ref_h * torch.rsqrt(ref_h.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
        torch.testing.assert_close(h.float(), ref_h, atol=6e-2, rtol=2e-2)
        torch.testing.assert_close(y.float(), ref_y, atol=6e-2, rtol=2e-2)
    comm.close()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(128, 256, 256), (300, 384, 1024), (1024, 4096, 4096), (64, 512, 640)])
def test_fp8_blockscaled_gemm(M, N, K):
    """Block-scaled e4m3 GEMM against the fp32 product of the dequantised operands."""
    from relax_b200 import ops
    from relax_b200.ops import cuda as C

    dev = "cuda"
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
    wq, ws = ops.blockwise_cast_to_fp8(w, 128)
    xq, xs = C.quantize_rows_fp8(x)
    y = C.fp8_linear(x, wq, ws, xq, xs)
    C.check_error_flag()
    kb = (K + 127) // 128
    xd = (torch.nn.functional.pad(xq.float(), (0, kb * 128 - K)).view(M, kb, 128) * xs.unsqueeze(-1)).view(M, -1)[:, :K]
    wd = ops.blockwise_dequant_fp8(wq, ws, 128, torch.float32)
    ref = xd @ wd.float().t()
    torch.testing.assert_close(y.float(), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
    # and the quantisation itself stays close to the bf16 product
    full = x.float() @ w.float().t()
    assert float((y.float() - full).abs().max()) < 0.12 * float(full.abs().max())
