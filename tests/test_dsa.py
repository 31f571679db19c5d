"""Sparse-attention ops of the DSA family: indexer logits, top-k, sparse MLA vs. dense, indexer loss (CPU)."""
import torch

from relax_b200.models import dsa as D


def test_indexer_logits_and_topk():
    torch.manual_seed(0)
    S, Hi, Dd = 6, 3, 4
    q, k, w = torch.randn(S, Hi, Dd), torch.randn(S, Dd), torch.rand(S, Hi)
    starts, ends = torch.tensor([0, 0, 0, 3, 3, 3]), torch.tensor([1, 2, 3, 4, 5, 6])
    lg = D.indexer_logits(q, k, w, starts, ends)
    ref = sum(w[2, h] * torch.relu(q[2, h] @ k[1]) for h in range(Hi))
    assert torch.allclose(lg[2, 1], ref, atol=1e-6)
    assert torch.isinf(lg[2, 3]) and torch.isinf(lg[4, 2]) and torch.isinf(lg[4, 5]) and torch.isfinite(lg[4, 4])
    idx = D.topk_indices(lg, 2)
    assert idx[0].tolist() == [0, -1] and set(idx[5].tolist()) <= {3, 4, 5} and idx.shape == (6, 2)
    assert D.topk_indices(lg, 8).shape == (6, 8) and (D.topk_indices(lg, 8)[:, 6:] == -1).all()
    s2, e2 = D.causal_ranges(torch.tensor([0, 3, 6], dtype=torch.int32), 6)
    assert s2.tolist() == starts.tolist() and e2.tolist() == ends.tolist()


def test_sparse_equals_dense_when_topk_covers_everything_and_handles_empty_rows():
    torch.manual_seed(1)
    S, H, Dq, dv = 10, 4, 12, 8
    q, kv = torch.randn(S, H, Dq), torch.randn(S, Dq)
    starts, ends = D.causal_ranges(torch.tensor([0, 4, 10], dtype=torch.int32), S)
    full = D.topk_indices(D.indexer_logits(torch.randn(S, 2, 3), torch.randn(S, 3), torch.rand(S, 2), starts, ends), S)
    o_s, lse = D.sparse_mla_attention(q, kv, full, dv, rows_per_chunk=3)
    o_d, p = D.dense_mla_attention(q, kv, starts, ends, dv)
    assert torch.allclose(o_s, o_d, atol=1e-5) and torch.isfinite(lse).all()
    assert torch.allclose(p.sum(-1), torch.ones(S, H), atol=1e-5)
    # picking the two best keys keeps most of a peaked distribution; an empty row gives zeros
    idx = torch.full((S, 2), -1)
    idx[3] = torch.tensor([1, 2])
    o2, lse2 = D.sparse_mla_attention(q, kv, idx, dv)
    assert float(o2[0].abs().sum()) == 0 and torch.isinf(lse2[0]).all() and torch.isfinite(lse2[3]).all()
    sc = (q[3] @ kv[[1, 2]].T) * Dq ** -0.5
    assert torch.allclose(o2[3], torch.softmax(sc, -1) @ kv[[1, 2], :dv], atol=1e-5)


def test_gradients_flow_to_q_and_selected_kv_only():
    torch.manual_seed(2)
    q = torch.randn(5, 2, 6, requires_grad=True)
    kv = torch.randn(5, 6, requires_grad=True)
    idx = torch.tensor([[0, -1], [0, 1], [1, 2], [0, 3], [4, 2]])
    out, _ = D.sparse_mla_attention(q, kv, idx, 4)
    out.square().sum().backward()
    assert torch.isfinite(q.grad).all() and float(q.grad[1].abs().sum()) > 0
    # row 0 attends one key: softmax is constant there, so only the value path carries gradient to kv[0]
    assert float(kv.grad[0, :4].abs().sum()) > 0


def test_indexer_loss_decreases_and_module_runs_sparse_and_dense():
    torch.manual_seed(3)
    m = D.DSAAttention(hidden=32, heads=2, topk=6)
    x = torch.randn(24, 32)
    pos = torch.cat([torch.arange(10), torch.arange(14)])
    cu = torch.tensor([0, 10, 24], dtype=torch.int32)
    y_sparse = m(x, pos, cu)
    m.topk = 64
    y_full, y_dense = m(x, pos, cu), m(x, pos, cu, dense=True)
    assert y_sparse.shape == (24, 32) and torch.allclose(y_full, y_dense, atol=1e-5) and not torch.allclose(y_sparse, y_dense, atol=1e-5)
    m.topk = 6
    opt = torch.optim.Adam(m.indexer.parameters(), lr=2e-2)
    losses = []
    for _ in range(25):
        _, kl, idx = m(x, pos, cu, return_aux=True)
        opt.zero_grad()
        kl.backward()
        opt.step()
        losses.append(float(kl))
    assert losses[-1] < losses[0] and idx.shape == (24, 6)
    assert m.linear_proj.weight.grad is None          # the indexer loss does not touch the trunk
