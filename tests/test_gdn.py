"""Gated delta rule: chunked form against the token-by-token recurrence; the GDN mixer layer (CPU)."""
import torch

from relax_b200.models.gdn import (GatedDeltaNet, causal_conv1d_varlen, gated_delta_rule_chunked,
                                   gated_delta_rule_recurrent, gated_delta_rule_varlen)


def _inputs(T, H=3, dk=8, dv=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H, dk, generator=g)
    k = torch.nn.functional.normalize(torch.randn(T, H, dk, generator=g), dim=-1)
    v = torch.randn(T, H, dv, generator=g)
    gl = -torch.rand(T, H, generator=g) * 0.5
    beta = torch.rand(T, H, generator=g)
    return q, k, v, gl, beta


def test_chunked_matches_recurrence_and_carries_state():
    q, k, v, g, b = _inputs(150)
    o_ref, s_ref = gated_delta_rule_recurrent(q, k, v, g, b)
    for chunk in (16, 64):
        o, s = gated_delta_rule_chunked(q, k, v, g, b, chunk)
        assert torch.allclose(o, o_ref, atol=2e-4), (o - o_ref).abs().max()
        assert torch.allclose(s, s_ref, atol=2e-4)
    # split in two calls with the state carried over
    o1, s1 = gated_delta_rule_chunked(q[:70], k[:70], v[:70], g[:70], b[:70], 32)
    o2, s2 = gated_delta_rule_chunked(q[70:], k[70:], v[70:], g[70:], b[70:], 32, state=s1)
    assert torch.allclose(torch.cat([o1, o2]), o_ref, atol=2e-4) and torch.allclose(s2, s_ref, atol=2e-4)


def test_gradients_match_recurrence():
    q, k, v, g, b = _inputs(40, seed=1)
    leaves = [x.clone().requires_grad_(True) for x in (q, k, v, g, b)]
    gated_delta_rule_recurrent(*leaves)[0].square().sum().backward()
    ref = [x.grad.clone() for x in leaves]
    leaves2 = [x.clone().requires_grad_(True) for x in (q, k, v, g, b)]
    gated_delta_rule_chunked(*leaves2, chunk=16)[0].square().sum().backward()
    for a, r in zip(leaves2, ref):
        assert torch.allclose(a.grad, r, atol=5e-4, rtol=1e-3)


def test_varlen_restarts_state_and_conv_stays_inside_sequences():
    q, k, v, g, b = _inputs(50, seed=2)
    cu = torch.tensor([0, 20, 50], dtype=torch.int32)
    o = gated_delta_rule_varlen(q, k, v, g, b, cu, chunk=16)
    assert torch.allclose(o[:20], gated_delta_rule_recurrent(q[:20], k[:20], v[:20], g[:20], b[:20])[0], atol=2e-4)
    assert torch.allclose(o[20:], gated_delta_rule_recurrent(q[20:], k[20:], v[20:], g[20:], b[20:])[0], atol=2e-4)
    x = torch.randn(50, 5)
    w = torch.randn(5, 4)
    y = causal_conv1d_varlen(x, w, cu)
    def ref(seg):
        pad = torch.cat([torch.zeros(3, 5), seg])
        return torch.nn.functional.silu(sum(pad[j:j + len(seg)] * w[:, j] for j in range(4)))
    assert torch.allclose(y[:20], ref(x[:20]), atol=1e-5) and torch.allclose(y[20:], ref(x[20:]), atol=1e-5)


def test_mixer_layer_chunked_equals_recurrent_and_trains():
    torch.manual_seed(0)
    m = GatedDeltaNet(hidden_size=32, num_k_heads=2, num_v_heads=4, head_k_dim=8, head_v_dim=8, chunk=16)
    x = torch.randn(45, 32)
    cu = torch.tensor([0, 13, 45], dtype=torch.int32)
    a, b = m(x, cu), m(x, cu, recurrent=True)
    assert a.shape == (45, 32) and torch.allclose(a, b, atol=2e-4)
    # the second sequence does not see the first
    alone = m(x[13:], torch.tensor([0, 32], dtype=torch.int32))
    assert torch.allclose(a[13:], alone, atol=2e-4)
    a.square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters())


def _cp_worker(rank, world):
    from relax_b200.parallel.cp import run_on_full_sequence, zigzag_rows
    from relax_b200.parallel.state import ParallelDims, init_parallel_state

    ps = init_parallel_state(ParallelDims(cp=2))
    torch.manual_seed(0)
    m = GatedDeltaNet(hidden_size=16, num_k_heads=2, num_v_heads=2, head_k_dim=8, head_v_dim=8, chunk=8)
    x_full = torch.randn(24, 16, generator=torch.Generator().manual_seed(5))
    rows = zigzag_rows(2, rank, 6)
    x_loc = x_full[rows].clone().requires_grad_(True)
    cu = torch.tensor([0, 24], dtype=torch.int32)
    y = run_on_full_sequence(lambda full: m(full, cu), x_loc, ps.cp)
    y.square().sum().backward()
    return rows, y.detach(), x_loc.grad.clone(), m.out_proj.weight.grad.clone()


def test_gdn_under_context_parallelism_matches_single_rank():
    from tests._mp import run_distributed

    outs = run_distributed(_cp_worker, 2)
    torch.manual_seed(0)
    m = GatedDeltaNet(hidden_size=16, num_k_heads=2, num_v_heads=2, head_k_dim=8, head_v_dim=8, chunk=8)
    x = torch.randn(24, 16, generator=torch.Generator().manual_seed(5)).requires_grad_(True)
    y = m(x, torch.tensor([0, 24], dtype=torch.int32))
    y.square().sum().backward()
    wsum = 0
    for rows, yl, gx, gw in outs:
        assert torch.allclose(yl, y.detach()[rows], atol=1e-5)
        assert torch.allclose(gx, x.grad[rows], atol=1e-4)
        wsum = wsum + gw
    assert torch.allclose(wsum, m.out_proj.weight.grad, atol=1e-4)     # parameter gradients add up over the CP ranks
