"""sm_100a kernels against plain PyTorch fp32 references of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _C():
    from relax_b200.ops import cuda as C

    assert C.available(), "the in-tree extension must be built and loadable on a GPU machine"
    return C


def _close(a, b, atol, rtol):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4e} (allowed {tol.max().item():.4e})"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (200, 328, 136), (1, 4096, 1024), (77, 152, 4096),
                                   (4096, 4096, 4096), (1024, 12288, 4096), (384, 32, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_nt(M, N, K, dtype):
    C = _C()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    b = torch.randn(N, K, device="cuda", generator=g).to(dtype)
    out = C.matmul_nt(a, b)
    ref = a.float() @ b.float().t()
    # two units in the last place of the 16-bit output (relative 2^-7 for bf16), plus a small absolute term for
    # outputs near zero, where the fp32 accumulation order shows
    _close(out, ref, atol=0.002 * math.sqrt(K), rtol=2.0 ** -7)
    C.check_error_flag()


@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (1000, 1000, 520), (5120, 4096, 4096), (384, 12288 + 64, 264)])
def test_gemm_pair_and_single_cta_kernels_agree_with_fp32(M, N, K, pair):
    """The CTA-pair kernel (cta_group::2, TMA-store epilogue) and the single-CTA kernel on the same problems, in the
    three operand layouts the trainer uses (forward, input gradient, weight gradient with fp32 accumulation)."""
    C = _C()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    dy = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm_raw(a, b, out, M, N, K, K, K, N, pair=pair)
    _close(out, a.float() @ b.float().t(), atol=0.002 * math.sqrt(K), rtol=2.0 ** -7)
    dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    C.gemm_raw(dy, b, dx, M, K, N, N, K, K, b_mn=True, pair=pair)          # dy @ b
    _close(dx, dy.float() @ b.float(), atol=0.002 * math.sqrt(N), rtol=2.0 ** -7)
    dw = torch.full((N, K), 0.5, device="cuda")
    C.gemm_raw(dy, a, dw, N, K, M, N, K, K, a_mn=True, b_mn=True, accumulate=True, pair=pair)     # += dy^T @ a
    _close(dw, dy.float().t() @ a.float() + 0.5, atol=2e-3 * math.sqrt(M), rtol=1e-4)
    C.check_error_flag()


@pytest.mark.parametrize("bn", [32, 64, 128, 256])
def test_gemm_every_tile_width(bn):
    C = _C()
    g = torch.Generator(device="cuda").manual_seed(bn)
    M, N, K = 300, 520, 264
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm_raw(a, b, out, M, N, K, K, K, N, force_bn=bn)
    _close(out, a.float() @ b.float().t(), atol=0.4, rtol=1e-2)
    C.check_error_flag()


def test_gemm_bias_fp32_out_and_accumulate():
    C = _C()
    g = torch.Generator(device="cuda").manual_seed(0)
    M, N, K = 256, 384, 256
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    bias = torch.randn(N, device="cuda", generator=g).bfloat16()
    ref = a.float() @ b.float().t()
    _close(C.matmul_nt(a, b, bias), ref + bias.float(), atol=0.4, rtol=1e-2)
    acc = torch.full((M, N), 3.0, device="cuda")
    C.matmul_nt(a, b, out=acc, accumulate=True)
    _close(acc, ref + 3.0, atol=1e-2, rtol=1e-3)
    o32 = C.matmul_nt(a, b, out_dtype=torch.float32)
    _close(o32, ref, atol=1e-2, rtol=1e-3)


def test_gemm_transposed_operands():
    C = _C()
    assert C.mn_major_ok(), "MN-major operand descriptors do not reproduce the K-major result"
    g = torch.Generator(device="cuda").manual_seed(3)
    M, N, K = 384, 640, 520
    dy = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    w = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    _close(C.matmul_nn(dy, w), dy.float() @ w.float(), atol=0.6, rtol=1e-2)          # dgrad
    _close(C.matmul_tn(dy, x), dy.float().t() @ x.float(), atol=0.6, rtol=1e-2)      # wgrad
    C.check_error_flag()


def test_linear_autograd():
    from relax_b200 import ops

    _C()
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(3, 100, 256, device="cuda", generator=g).bfloat16().requires_grad_()
    w = (torch.randn(512, 256, device="cuda", generator=g) * 0.05).bfloat16().requires_grad_()
    y = ops.linear(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(dy.float())
    _close(y, yr, 0.05, 1e-2)
    _close(x.grad, xr.grad, 0.05, 2e-2)
    _close(w.grad, wr.grad, 0.3, 2e-2)


@pytest.mark.parametrize("rows,cols", [(1000, 4096), (2304, 4096), (37, 1024), (5000, 128), (16, 8192)])
def test_rmsnorm_fwd_bwd(rows, cols):
    from relax_b200 import ops
    from relax_b200.ops import reference as R

    _C()
    g = torch.Generator(device="cuda").manual_seed(rows)
    x = torch.randn(rows, cols, device="cuda", generator=g).bfloat16().requires_grad_()
    res = torch.randn(rows, cols, device="cuda", generator=g).bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).bfloat16().requires_grad_()
    y = ops.rmsnorm(x, w, 1e-6)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yf = R.rmsnorm(xf, wf, 1e-6)
    yf.backward(dy.float())
    _close(y, yf, 0.02, 1e-2)
    _close(x.grad, xf.grad, 0.03, 2e-2)
    _close(w.grad, wf.grad, 0.02 * math.sqrt(rows), 2e-2)
    # fused residual add
    x.grad = None
    w.grad = None
    y2, r2 = ops.add_rmsnorm(x, res, w, 1e-6)
    (y2.float().sum() + 2 * r2.float().sum()).backward()
    xf2, rf2 = x.detach().float().requires_grad_(), res.detach().float().requires_grad_()
    rsum = (xf2 + rf2) + ((xf2 + rf2).bfloat16().float() - (xf2 + rf2)).detach()
    yr2 = R.rmsnorm(rsum, wf.detach(), 1e-6)
    (yr2.sum() + 2 * rsum.sum()).backward()
    _close(y2, yr2, 0.02, 1e-2)
    _close(r2, rsum, 0.02, 1e-2)
    _close(x.grad, xf2.grad, 0.05, 3e-2)
    _close(res.grad, rf2.grad, 0.05, 3e-2)


def test_rope_and_swiglu():
    from relax_b200 import ops
    from relax_b200.ops import reference as R

    _C()
    g = torch.Generator(device="cuda").manual_seed(5)
    T, H, D = 333, 12, 128
    x = torch.randn(T, H, D, device="cuda", generator=g).bfloat16().requires_grad_()
    pos = torch.randint(0, 5000, (T,), device="cuda", generator=g)
    cos, sin = R.rope_cos_sin(pos, D, 1e6)
    y = ops.apply_rope(x, cos, sin)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf = x.detach().float().requires_grad_()
    yf = R.apply_rope(xf, cos, sin)
    yf.backward(dy.float())
    _close(y, yf, 0.02, 1e-2)
    _close(x.grad, xf.grad, 0.02, 1e-2)
    gu = torch.randn(257, 2 * 1536, device="cuda", generator=g).bfloat16().requires_grad_()
    a = ops.swiglu(gu)
    da = torch.randn_like(a)
    a.backward(da)
    gf = gu.detach().float().requires_grad_()
    af = R.swiglu(gf)
    af.backward(da.float())
    _close(a, af, 0.02, 1e-2)
    _close(gu.grad, gf.grad, 0.03, 2e-2)


@pytest.mark.parametrize("split,grad_fp32", [(True, True), (True, False), (False, True)])
def test_fused_adam_matches_reference(split, grad_fp32):
    from relax_b200.ops.reference import adam_step
    from relax_b200.train.optimizer import _join_fp32, _split_fp32

    C = _C()
    n = 1 << 20
    g = torch.Generator(device="cuda").manual_seed(6)
    master = torch.randn(n, device="cuda", generator=g) * 0.02
    grad = torch.randn(n, device="cuda", generator=g) * 1e-3
    grad = grad if grad_fp32 else grad.bfloat16()
    p, rem = _split_fp32(master, torch.bfloat16)
    mst = rem.clone() if split else master.clone()
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    rm, rv, rp = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), master.clone()
    for step in (1, 2, 3):
        C.fused_adam(p, mst, grad, m, v, step, 1e-4, 0.9, 0.999, 1e-8, 0.01, 0.5, split)
        adam_step(rp, grad, rm, rv, step, 1e-4, 0.9, 0.999, 1e-8, 0.01, 0.5)
    got = _join_fp32(p, mst) if split else mst
    _close(got, rp, 1e-7, 1e-5)
    assert (p.float() - got).abs().max() <= got.abs().max() * 2 ** -8
    _close(m, rm, 1e-9, 1e-5)
    assert abs(C.sumsq(grad).item() - grad.float().pow(2).sum().item()) < 1e-3 * grad.float().pow(2).sum().item()


def test_copy_table_weight_sync_is_bit_exact():
    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel
    from relax_b200.rollout.weights import RolloutWeights
    from relax_b200.weight_sync.plan import TrainerLayout
    from relax_b200.weight_sync.sync import WeightSync, apply_block

    _C()
    cfg = get_config("tiny", dtype="bf16")
    model = GPTModel(cfg, device="cuda", seed=1)
    rw = RolloutWeights(cfg, 1, 0, "cuda", torch.bfloat16)
    ws = WeightSync(cfg, TrainerLayout(), 1, [0], [0])
    ws.update_weights(dict(model.named_parameters()), rw)
    exp = RolloutWeights(cfg, 1, 0, "cuda", torch.bfloat16)
    params = dict(model.named_parameters())
    for b in ws.plan:
        apply_block(b, params[b.src_name].detach(), exp.p[b.dst_name])
    assert torch.equal(rw.flat, exp.flat) and rw.flat.abs().sum() > 0


def test_quantisers():
    from relax_b200 import ops
    from relax_b200.ops import reference as R

    _C()
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(100, 200, device="cuda", generator=g)
    for bm, bn, sym in [(1, 32, True), (32, 1, True), (16, 16, False), (1, 32, False)]:
        o, s, z = ops.fake_int4_quant(x, bm, bn, sym)
        ro, rs, rz = R.fake_int4_quant(x, bm, bn, sym)
        _close(s, rs, 1e-6, 1e-5)
        _close(z, rz, 1e-6, 0)
        # rounding ties may differ by one step in a few places; everything else must agree
        bad = ((o - ro).abs() > 1e-5).float().mean().item()
        assert bad < 1e-3, bad
    w = torch.randn(300, 260, device="cuda", generator=g).bfloat16()
    for ue in (False, True):
        q, s = ops.blockwise_cast_to_fp8(w, 128, ue)
        rq, rs = R.blockwise_cast_to_fp8(w, 128, ue)
        _close(s, rs, 1e-9, 1e-5)
        d = ops.blockwise_dequant_fp8(q, s, 128)
        _close(d, w, 0.02, 0.07)
        assert (q.float() - rq.float()).abs().max() <= 32


def test_kv_scatter():
    C = _C()
    g = torch.Generator(device="cuda").manual_seed(8)
    T, H, D = 50, 4, 128
    qkv = torch.randn(T, (8 + 2 * H) * D, device="cuda", generator=g).bfloat16()
    k = qkv[:, 8 * D:(8 + H) * D].view(T, H, D)
    v = qkv[:, (8 + H) * D:].view(T, H, D)
    kc = torch.zeros(16 * 8, H, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(128, device="cuda", generator=g)[:T]
    C.kv_scatter(k, v, kc, vc, slots)
    assert torch.equal(kc[slots], k) and torch.equal(vc[slots], v)


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("Mt,N,K,S", [(16, 128, 256, 1), (64, 256, 512, 2), (100, 384, 1024, 4), (128, 4096, 4096, 0),
                                     (200, 256, 2048, 8), (256, 1024, 1024, 2), (130, 768, 2048, 0), (7, 136, 264, 1)])
def test_decode_gemm_cluster_splitk(Mt, N, K, S, swiglu):
    """Weight-streaming decode GEMM (weights as the MMA M operand, split-K reduced through distributed shared
    memory), with and without the SwiGLU epilogue, against fp32."""
    C = _C()
    L = C._load()
    if swiglu and (N // 2) % 64:
        pytest.skip("the SwiGLU variant takes 64 gate/up pairs per tile")
    g = torch.Generator(device="cuda").manual_seed(Mt + N + K + S)
    x = torch.randn(Mt, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    y = torch.full((Mt, N // 2 if swiglu else N), float("nan"), device="cuda", dtype=torch.bfloat16)
    assert L.decode_gemm(x, w, y, swiglu, S, C.err_flag(x.device)), "the shape is inside the kernel's range"
    C.check_error_flag(x.device)
    ref = x.float() @ w.float().t()
    if swiglu:
        F = N // 2
        ref = torch.nn.functional.silu(ref[:, :F]) * ref[:, F:]
    _close(y, ref, atol=0.002 * math.sqrt(K), rtol=2 ** -7)


@pytest.mark.parametrize("dual", [None, 3.0])
def test_fused_policy_loss_matches_eager(dual):
    from relax_b200.algo import ppo_utils as P

    g = torch.Generator(device="cuda").manual_seed(5)
    n = 100_003
    kl = (torch.randn(n, device="cuda", generator=g) * 0.3).requires_grad_(True)
    adv = torch.randn(n, device="cuda", generator=g)
    w = torch.rand(n, device="cuda", generator=g)
    loss, clip = _C().policy_loss(kl, adv, 0.2, 0.28, dual)
    (loss * w).sum().backward()
    g_fused, kl.grad = kl.grad.clone(), None
    # the eager statement of the same loss (CPU path of compute_policy_loss)
    ratio = torch.exp(-kl)
    l1, l2 = -ratio * adv, -ratio.clamp(0.8, 1.28) * adv
    ref = torch.maximum(l1, l2)
    if dual is not None:
        ref = torch.where(adv < 0, torch.minimum(-dual * adv, ref), ref)
    (ref * w).sum().backward()
    _close(loss, ref, 1e-5, 1e-5)
    assert torch.equal(clip, (l2 > l1).float())
    _close(g_fused, kl.grad, 1e-5, 1e-5)
    # and the public entry point takes the fused path on a GPU
    out, _ = P.compute_policy_loss(kl.detach(), adv, 0.2, 0.28, dual)
    _close(out, ref, 1e-5, 1e-5)
