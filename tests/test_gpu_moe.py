"""Grouped (per-expert) GEMM kernels and the MoE layer on the GPU against fp32 statements of the same math."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, atol, rtol, what=""):
    err = (a.float() - b.float()).abs()
    tol = atol + rtol * b.float().abs()
    assert bool((err <= tol).all()), f"{what}: max err {err.max().item():.4e}"


@pytest.mark.parametrize("E,N,K,counts", [(4, 256, 128, [100, 0, 300, 17]), (16, 1536, 2048, None), (3, 192, 320, [1, 129, 128])])
def test_grouped_linear_forward_backward(E, N, K, counts):
    from relax_b200 import ops
    from relax_b200.models.moe import padded_expert_layout
    from relax_b200.ops import cuda as C

    assert C.available()
    g = torch.Generator(device="cuda").manual_seed(E + N + K)
    if counts is None:
        counts = torch.randint(0, 400, (E,), generator=torch.Generator().manual_seed(1)).tolist()
    e_of = torch.cat([torch.full((c,), e, dtype=torch.int64) for e, c in enumerate(counts)]).cuda()
    e_of = e_of[torch.randperm(e_of.numel(), device="cuda", generator=g)]        # unsorted rows
    R = e_of.numel()
    x = torch.randn(R, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(E, N, K, device="cuda", generator=g) * 0.05).bfloat16().requires_grad_()
    order, dest, cap, tile_expert, expert_rows = padded_expert_layout(e_of, E)
    xp = x.new_zeros(cap, K).index_copy(0, dest, x[order]).requires_grad_()
    y = ops.grouped_linear(xp, w, tile_expert, expert_rows)
    inv = torch.empty_like(order)
    inv[order] = dest
    got = y[inv]
    ref = torch.einsum("rk,rnk->rn", x.float(), w.float()[e_of])
    _close(got, ref, 0.002 * math.sqrt(K), 2.0 ** -7, "forward")
    assert float(y.float().abs().sum() - got.float().abs().sum()) < 1e-3 * max(1.0, float(got.float().abs().sum()))   # padding rows are zero
    dy_rows = torch.randn(R, N, device="cuda", generator=g).bfloat16()
    dyp = torch.zeros(cap, N, device="cuda", dtype=torch.bfloat16).index_copy(0, dest, dy_rows[order])
    y.backward(dyp)
    dx_ref = torch.einsum("rn,rnk->rk", dy_rows.float(), w.float()[e_of])
    _close(xp.grad[inv], dx_ref, 0.002 * math.sqrt(N), 2.0 ** -7, "dgrad")
    dw_ref = torch.zeros(E, N, K, device="cuda")
    dw_ref.index_add_(0, e_of, torch.einsum("rn,rk->rnk", dy_rows.float(), x.float())) if R * N * K < 5e8 else None
    if R * N * K < 5e8:
        _close(w.grad, dw_ref, 0.01 * math.sqrt(max(counts)), 2.0 ** -6, "wgrad")
    else:        # large case: compare per expert
        for e in range(E):
            m = e_of == e
            _close(w.grad[e], dy_rows[m].float().t() @ x[m].float(), 0.01 * math.sqrt(max(counts)), 2.0 ** -6, f"wgrad expert {e}")
    # accumulation into an fp32 main_grad
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.full((E, N, K), 0.25, device="cuda")
    ops.grouped_linear(xp.detach(), w2, tile_expert, expert_rows).backward(dyp)
    assert w2.grad is None
    _close(w2.main_grad - 0.25, w.grad, 0.02 * math.sqrt(max(counts)), 2.0 ** -6, "wgrad accumulate")
    C.check_error_flag()


def test_moe_layer_matches_cpu_statement():
    """The whole MoE MLP (router, permutation, grouped expert GEMMs, weighted combine) on the GPU in bf16 against the
    same layer evaluated in fp32 on the CPU, forward and parameter gradients."""
    import dataclasses

    from relax_b200.models.config import get_config
    from relax_b200.models.moe import MoEMLP
    from relax_b200.models.transformer import ParamInit
    from relax_b200.parallel.state import single_process_state

    cfg = dataclasses.replace(get_config("tiny-moe"), hidden_size=256, moe_ffn_hidden_size=128, num_experts=8, moe_top_k=2)
    ps = single_process_state()
    ref = MoEMLP(cfg, ps, torch.float32, "cpu", ParamInit(3, "cpu"), 0)
    gpu = MoEMLP(cfg, ps, torch.bfloat16, "cuda", ParamInit(3, "cuda"), 0).cuda()
    with torch.no_grad():
        for (n, p), (_, q) in zip(gpu.named_parameters(), ref.named_parameters()):
            p.copy_(q.to(p.dtype))
            q.copy_(p.float().cpu())          # the reference uses the bf16-rounded weights
    x = (torch.randn(300, cfg.hidden_size, generator=torch.Generator().manual_seed(0)) * 0.5).bfloat16()
    xr = x.float().requires_grad_()
    xg = x.cuda().requires_grad_()
    yr = ref(xr)
    yg = gpu(xg)
    _close(yg.cpu(), yr, 2e-2, 2e-2, "moe forward")
    dy = torch.randn(yr.shape, generator=torch.Generator().manual_seed(1)) * 0.1
    yr.backward(dy)
    yg.backward(dy.cuda().bfloat16())
    _close(xg.grad.cpu(), xr.grad, 2e-2, 5e-2, "moe dx")
    _close(gpu.experts.linear_fc2.weight.grad.cpu(), ref.experts.linear_fc2.weight.grad, 2e-2, 5e-2, "moe dW2")
