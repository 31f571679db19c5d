"""Tensor-core attention, rollout kernels and the fused LM head against fp32 PyTorch references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _C():
    from relax_b200.ops import cuda as C

    assert C.available()
    return C


def _close(a, b, atol, rtol, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"{what}: max err {err.max().item():.4e} at tol {tol.max().item():.4e}"


def _mk(lens_q, lens_k, Hq, Hkv, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    Tq, Tk = sum(lens_q), sum(lens_k)
    q = torch.randn(Tq, Hq, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(Tk, Hkv, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(Tk, Hkv, 128, device="cuda", generator=g).bfloat16()
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device="cuda")
    return q, k, v, cu_q, cu_k


@pytest.mark.parametrize("lens,Hq,Hkv,causal", [
    ([128], 2, 2, True), ([64], 4, 1, True), ([300, 17, 129, 1], 8, 2, True), ([1000], 4, 4, True),
    ([257, 511], 4, 2, False), ([2048, 77], 8, 2, True),
])
def test_flash_attention_forward(lens, Hq, Hkv, causal):
    from relax_b200 import ops
    from relax_b200.ops import reference as R

    C = _C()
    q, k, v, cu, _ = _mk(lens, lens, Hq, Hkv, sum(lens))
    o = ops.attention_varlen(q, k, v, cu, causal=causal)
    ref = R.attention_varlen(q.float(), k.float(), v.float(), cu, causal=causal)
    _close(o, ref, 2e-2, 2e-2, "fwd")
    C.check_error_flag()


def test_flash_attention_query_shorter_than_keys():
    """Chunked prefill / CP layout: queries are the tail of the key sequence (bottom-right causal)."""
    from relax_b200 import ops
    from relax_b200.ops import reference as R

    C = _C()
    q, k, v, cu_q, cu_k = _mk([100, 64], [400, 64], 4, 2, 5)
    o = ops.attention_varlen(q, k, v, cu_q, causal=True, cu_seqlens_k=cu_k)
    ref = R.attention_varlen(q.float(), k.float(), v.float(), cu_q, causal=True, cu_seqlens_k=cu_k)
    _close(o, ref, 2e-2, 2e-2, "fwd q<k")
    C.check_error_flag()


@pytest.mark.parametrize("lens,Hq,Hkv,causal", [
    ([128], 1, 1, True), ([64], 2, 1, True), ([300, 17, 129], 4, 2, True), ([640], 8, 2, True), ([257, 100], 2, 2, False),
])
def test_flash_attention_backward(lens, Hq, Hkv, causal):
    from relax_b200 import ops
    from relax_b200.ops import reference as R

    C = _C()
    q, k, v, cu, _ = _mk(lens, lens, Hq, Hkv, 7 + sum(lens))
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    o = ops.attention_varlen(q, k, v, cu, causal=causal)
    do = torch.randn_like(o)
    o.backward(do)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    of = R.attention_varlen(qf, kf, vf, cu, causal=causal)
    of.backward(do.float())
    _close(q.grad, qf.grad, 4e-2, 4e-2, "dq")
    _close(k.grad, kf.grad, 4e-2 * math.sqrt(Hq // Hkv), 4e-2, "dk")
    _close(v.grad, vf.grad, 4e-2 * math.sqrt(Hq // Hkv), 4e-2, "dv")
    C.check_error_flag()


@pytest.mark.parametrize("B,Hq,Hkv,bs,maxctx", [(3, 8, 2, 16, 700), (64, 32, 8, 16, 300), (2, 28, 4, 32, 5000), (5, 4, 4, 16, 40)])
def test_paged_decode_attention(B, Hq, Hkv, bs, maxctx):
    from relax_b200 import ops
    from relax_b200.ops import reference as R

    _C()
    g = torch.Generator(device="cuda").manual_seed(B)
    ctx = torch.randint(1, maxctx + 1, (B,), device="cuda", generator=g)
    ctx[0] = maxctx
    nb_per = (maxctx + bs - 1) // bs
    nblocks = B * nb_per + 3
    kc = torch.randn(nblocks, bs, Hkv, 128, device="cuda", generator=g).bfloat16()
    vc = torch.randn(nblocks, bs, Hkv, 128, device="cuda", generator=g).bfloat16()
    bt = torch.randperm(nblocks, device="cuda", generator=g)[: B * nb_per].view(B, nb_per).int()
    q = torch.randn(B, Hq, 128, device="cuda", generator=g).bfloat16()
    o = ops.paged_decode_attention(q, kc, vc, bt, ctx)
    ref = R.paged_decode_attention(q.float(), kc.float(), vc.float(), bt, ctx)
    _close(o, ref, 2e-2, 2e-2, "decode")


def test_sampling_matches_reference_and_distribution():
    from relax_b200 import ops
    from relax_b200.ops import reference as R

    _C()
    g = torch.Generator(device="cuda").manual_seed(0)
    B, V = 64, 151936
    logits = torch.randn(B, V, device="cuda", generator=g) * 3
    u = torch.rand(B, device="cuda", generator=g)
    for temp, k, p in [(1.0, -1, 1.0), (0.7, 50, 1.0), (1.0, -1, 0.9), (1.3, 100, 0.8), (0.0, -1, 1.0)]:
        t = torch.full((B,), temp, device="cuda")
        tk = torch.full((B,), k, device="cuda", dtype=torch.int64)
        tp = torch.full((B,), p, device="cuda")
        tok, lp = ops.sample(logits, t, tk, tp, u)
        rtok, rlp = R.sample(logits, t, tk, tp, u)
        agree = (tok == rtok).float().mean().item()
        assert agree >= 0.95, (temp, k, p, agree)
        same = tok == rtok
        _close(lp[same], rlp[same], 1e-3, 1e-4, "sample logp")
        if k > 0:   # every sampled token is inside the top-k set
            topk = logits.topk(k, -1).indices
            assert bool((topk == tok[:, None]).any(-1).all())
    # empirical distribution of many draws from one small row
    row = torch.tensor([[2.0, 1.0, 0.0, -1.0]], device="cuda").repeat(4096, 1)
    uu = torch.rand(4096, device="cuda", generator=g)
    tok, _ = ops.sample(row, torch.ones(4096, device="cuda"), torch.full((4096,), -1, device="cuda"),
                        torch.ones(4096, device="cuda"), uu)
    freq = torch.bincount(tok, minlength=4).float() / 4096
    assert (freq - torch.softmax(row[0], -1)).abs().max() < 0.03


def test_topk_router_forward_backward():
    from relax_b200 import ops
    from relax_b200.ops import reference as R

    _C()
    g = torch.Generator(device="cuda").manual_seed(1)
    for E, K, norm in [(128, 8, True), (8, 2, True), (64, 6, False)]:
        z = torch.randn(333, E, device="cuda", generator=g).requires_grad_()
        w, idx, probs = ops.topk_router(z, K, norm)
        zr = z.detach().clone().requires_grad_()
        rw, ridx, rp = R.topk_router(zr, K, norm)
        assert torch.equal(idx, ridx)
        _close(w, rw, 1e-6, 1e-5)
        _close(probs, rp, 1e-7, 1e-5)
        gw = torch.randn_like(w)
        gp = torch.randn_like(probs) * 0.1
        (w * gw).sum().backward(retain_graph=True)
        (rw * gw).sum().backward(retain_graph=True)
        _close(z.grad, zr.grad, 1e-6, 1e-4)
        z.grad = None
        zr.grad = None
        ((w * gw).sum() + (probs * gp).sum()).backward()
        ((rw * gw).sum() + (rp * gp).sum()).backward()
        _close(z.grad, zr.grad, 1e-6, 1e-4)


@pytest.mark.parametrize("T,V,H,temp", [(300, 1000, 256, 1.0), (1111, 151936 // 8, 512, 0.7), (5000, 2048, 128, 1.0)])
def test_fused_lm_head_logprob_entropy(T, V, H, temp):
    from relax_b200 import ops

    C = _C()
    g = torch.Generator(device="cuda").manual_seed(T)
    h = torch.randn(T, H, device="cuda", generator=g).bfloat16().requires_grad_()
    w = (torch.randn(V, H, device="cuda", generator=g) * 0.05).bfloat16().requires_grad_()
    tgt = torch.randint(0, V, (T,), device="cuda", generator=g)
    lp, en = ops.fused_lm_head_logprob(h, w, tgt, None, 0, True, temp)
    glp, gen = torch.randn_like(lp), torch.randn_like(en) * 0.1
    (lp * glp + en * gen).sum().backward()
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    z = (hf @ wf.t()) / temp
    ls = torch.log_softmax(z, -1)
    rlp = ls.gather(-1, tgt[:, None])[:, 0]
    ren = -(ls.exp() * ls).sum(-1)
    (rlp * glp + ren * gen).sum().backward()
    _close(lp, rlp, 2e-2, 1e-2, "logp")
    _close(en, ren, 2e-2, 1e-2, "entropy")
    _close(h.grad, hf.grad, 2e-2, 5e-2, "dh")
    _close(w.grad, wf.grad, 3e-2, 5e-2, "dW")
    C.check_error_flag()


def test_fused_lm_head_vocab_shard_offsets():
    """Targets outside the local vocabulary shard contribute -inf (not found) partials."""
    from relax_b200.ops import cuda as C

    _C()
    g = torch.Generator(device="cuda").manual_seed(9)
    T, V, H = 200, 512, 128
    h = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    w = (torch.randn(V, H, device="cuda", generator=g) * 0.1).bfloat16()
    tgt = torch.randint(0, V, (T,), device="cuda", generator=g)
    full_lp, full_en = C.fused_lm_head_logprob(h, w, tgt)
    # two shards combined by hand the way the TP all-reduces do
    parts = []
    for r in range(2):
        sp = C._load().lm_head_splits(T, V // 2)
        part = torch.empty(T, sp, 4, device="cuda")
        C._load().lm_head_logprob(h, w[r * V // 2:(r + 1) * V // 2].contiguous(), tgt, part, r * V // 2, 1.0, sp,
                                  C.err_flag())
        parts.append(part)
    part = torch.cat(parts, 1)
    m = part[..., 0].max(1).values
    sc = torch.exp(part[..., 0] - m[:, None])
    s = (part[..., 1] * sc).sum(1)
    zt = part[..., 3].max(1).values
    assert torch.isfinite(zt).all()
    _close(zt - (m + torch.log(s)), full_lp, 1e-4, 1e-4)


@pytest.mark.parametrize("D,causal", [(64, True), (80, False), (96, True)])
def test_flash_attention_narrow_heads_are_padded_to_the_kernel_width(D, causal):
    """head_dim 64 / 80 / 96 (ViT towers, small models) run through the head_dim-128 tensor-core kernels by zero
    padding; forward and backward against the fp32 statement."""
    from relax_b200 import ops
    from relax_b200.ops import reference as R

    C = _C()
    lens, Hq, Hkv = [300, 77, 129], 4, 2
    g = torch.Generator(device="cuda").manual_seed(D)
    T = sum(lens)
    q, k, v = (torch.randn(T, h, D, device="cuda", generator=g).bfloat16().requires_grad_() for h in (Hq, Hkv, Hkv))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    launches = C._load().launch_count() if hasattr(C._load(), "launch_count") else None
    o = ops.attention_varlen(q, k, v, cu, causal=causal)
    assert o.shape == (T, Hq, D)
    do = torch.randn_like(o)
    o.backward(do)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    of = R.attention_varlen(qf, kf, vf, cu, causal=causal)
    of.backward(do.float())
    _close(o, of, 2e-2, 2e-2, "o")
    _close(q.grad, qf.grad, 4e-2, 4e-2, "dq")
    _close(k.grad, kf.grad, 6e-2, 4e-2, "dk")
    _close(v.grad, vf.grad, 6e-2, 4e-2, "dv")
    if launches is not None:
        assert C._load().launch_count() > launches, "the tensor-core kernels ran (no PyTorch statement)"
    C.check_error_flag()


def test_vision_encoder_runs_on_the_gpu_kernels():
    """A Qwen2.5-VL style tower (head_dim 80, bias in qkv, 2-D rotary, windowless full attention per image) in bf16
    on the GPU against the same module in fp32 on the CPU."""
    from relax_b200.models.vision import VisionConfig, VisionEncoder

    _C()
    cfg = VisionConfig(depth=2, out_hidden_size=512)
    assert cfg.head_dim == 80
    cpu = VisionEncoder(cfg, dtype=torch.float32, device="cpu", seed=3)
    gpu = VisionEncoder(cfg, dtype=torch.bfloat16, device="cuda", seed=3)
    grid = torch.tensor([[1, 8, 12], [1, 4, 4]])
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(n, cfg.patch_dim, generator=torch.Generator().manual_seed(1))
    ref = cpu(px, grid)
    out = gpu(px.cuda(), grid.cuda())
    assert out.shape == ref.shape
    rel = (out.float().cpu() - ref).norm() / ref.norm()
    assert rel < 3e-2, f"relative error {rel:.3e}"
    out.float().sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in gpu.parameters())
