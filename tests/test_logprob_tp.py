"""Vocab-parallel log-prob/entropy and TP model parity on gloo worlds."""
import torch

from tests._mp import run_distributed


def _vp_worker(rank, world):
    import torch.distributed as dist
    from relax_b200.algo.logprob import vocab_parallel_log_probs_and_entropy, top_k_log_probs_on_ids

    torch.manual_seed(0)
    T, V = 13, 64
    full = torch.randn(T, V, dtype=torch.float64)
    tgt = torch.randint(0, V, (T,))
    gl, ge = torch.randn(T, dtype=torch.float64), torch.randn(T, dtype=torch.float64)
    ref = full.clone().requires_grad_()
    lsm = torch.log_softmax(ref / 0.7, -1)
    lp_ref = lsm.gather(-1, tgt[:, None])[:, 0]
    ent_ref = -(lsm.exp() * lsm).sum(-1)
    (lp_ref * gl + ent_ref * ge).sum().backward()
    vl = V // world
    loc = full[:, rank * vl:(rank + 1) * vl].clone().requires_grad_()
    lp, ent = vocab_parallel_log_probs_and_entropy(loc, tgt, dist.group.WORLD, rank * vl, True, 0.7)
    (lp.double() * gl + ent.double() * ge).sum().backward()
    assert torch.allclose(lp.double(), lp_ref, atol=1e-5)
    assert torch.allclose(ent.double(), ent_ref, atol=1e-5)
    assert torch.allclose(loc.grad, ref.grad[:, rank * vl:(rank + 1) * vl], atol=1e-5)
    ids = torch.randint(0, V, (T, 4))
    tk = top_k_log_probs_on_ids(full[:, rank * vl:(rank + 1) * vl].float(), ids, dist.group.WORLD, rank * vl)
    assert torch.allclose(tk.double(), torch.log_softmax(full, -1).gather(-1, ids), atol=1e-5)
    return True


def test_vocab_parallel_logprob_entropy_two_ranks():
    assert all(run_distributed(_vp_worker, 2))


def _tp_worker(rank, world, model_name):
    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel
    from relax_b200.parallel.state import ParallelDims, init_parallel_state, single_process_state

    cfg = get_config(model_name)
    ps = init_parallel_state(ParallelDims(tp=2))
    torch.manual_seed(0)
    T = 48
    tok = torch.randint(0, cfg.vocab_size, (T,))
    cu = torch.tensor([0, 20, 48], dtype=torch.int32)
    pos = torch.cat([torch.arange(20), torch.arange(28)])

    def run(model):
        h = model(tok, pos, cu)
        lp, en = model.log_probs(h[:-1], tok[1:], temperature=1.0)
        (lp.sum() + 0.1 * en.sum()).backward()
        return lp.detach(), en.detach()

    m1 = GPTModel(cfg, single_process_state(), seed=3)
    lp1, en1 = run(m1)
    m2 = GPTModel(cfg, ps, seed=3)
    lp2, en2 = run(m2)
    assert torch.allclose(lp1, lp2, atol=2e-4), (lp1 - lp2).abs().max()
    assert torch.allclose(en1, en2, atol=2e-4)
    # gradient of a row-parallel shard equals the matching slice of the full gradient
    g1 = m1.decoder.layers[0].mlp.linear_fc2.weight.grad if hasattr(m1.decoder.layers[0].mlp, "linear_fc2") else None
    if g1 is not None:
        g2 = m2.decoder.layers[0].mlp.linear_fc2.weight.grad
        n = g2.shape[1]
        assert torch.allclose(g1[:, rank * n:(rank + 1) * n], g2, atol=2e-4)
    # replicated norm weights need the TP all-reduce the optimizer performs
    import torch.distributed as dist
    gn = m2.decoder.layers[1].self_attention.linear_qkv.layer_norm_weight.grad.clone()
    dist.all_reduce(gn, group=ps.tp.group)
    assert torch.allclose(gn, m1.decoder.layers[1].self_attention.linear_qkv.layer_norm_weight.grad, atol=2e-4)
    return True


def test_tensor_parallel_model_matches_single():
    assert all(run_distributed(_tp_worker, 2, "tiny"))


def _ep_worker(rank, world):
    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel
    from relax_b200.parallel.state import ParallelDims, init_parallel_state, single_process_state

    cfg = get_config("tiny-moe")
    ps = init_parallel_state(ParallelDims(dp=2, ep=2))
    torch.manual_seed(rank)
    T = 32
    tok = torch.randint(0, cfg.vocab_size, (T,))
    cu = torch.tensor([0, T], dtype=torch.int32)
    pos = torch.arange(T)
    m1 = GPTModel(cfg, single_process_state(), seed=5)
    m2 = GPTModel(cfg, ps, seed=5)
    h1, h2 = m1(tok, pos, cu), m2(tok, pos, cu)
    assert torch.allclose(h1, h2, atol=2e-4), (h1 - h2).abs().max()
    h2.sum().backward()
    h1.sum().backward()
    return True


def test_expert_parallel_matches_single():
    assert all(run_distributed(_ep_worker, 2))
