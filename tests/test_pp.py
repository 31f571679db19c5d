"""1F1B pipeline schedule with a streaming micro-batch source equals single-process training (gloo, 2 stages)."""
import torch

from tests._mp import run_distributed


def _pp_worker(rank, world, n_mb):
    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel
    from relax_b200.parallel.pp import forward_backward_1f1b
    from relax_b200.parallel.state import ParallelDims, init_parallel_state, single_process_state

    cfg = get_config("tiny")
    ps = init_parallel_state(ParallelDims(pp=2))
    model = GPTModel(cfg, ps, seed=11)
    assert len(model.decoder.layers) == 1 and model.pre_process == (rank == 0) and model.post_process == (rank == 1)
    torch.manual_seed(0)
    mbs = []
    for i in range(n_mb):
        T = 16 + 4 * i
        mbs.append({"tokens": torch.randint(0, cfg.vocab_size, (T,)), "pos": torch.arange(T), "cu": torch.tensor([0, T], dtype=torch.int32)})

    # every stage needs tokens/positions of the micro-batch it works on: broadcast them as part of the stream
    counter = {"i": 0}

    def forward_step(mb, x):
        i = counter["i"]
        counter["i"] += 1
        b = mbs[i]                               # test shortcut: all ranks hold the synthetic data
        if rank == 0:
            h = model(b["tokens"], b["pos"], b["cu"])
            return h, None
        h = model(None, b["pos"], b["cu"], hidden_in=x)
        lp, _ = model.log_probs(h[:-1], b["tokens"][1:])
        return h, -lp.mean()

    def gen():
        for b in mbs:                            # a generator: the schedule cannot know its length in advance
            yield b

    losses = forward_backward_1f1b(gen() if rank == 0 else None, forward_step, ps.pp, "cpu", torch.float32)
    # single-process reference
    ref = GPTModel(cfg, single_process_state(), seed=11)
    ref_losses = []
    for b in mbs:
        h = ref(b["tokens"], b["pos"], b["cu"])
        lp, _ = ref.log_probs(h[:-1], b["tokens"][1:])
        l = -lp.mean()
        l.backward()
        ref_losses.append(l.detach())
    if rank == 1:
        assert len(losses) == n_mb
        assert torch.allclose(torch.stack(losses), torch.stack(ref_losses), atol=1e-5)
        g, gr = model.decoder.layers[0].mlp.linear_fc2.weight.grad, ref.decoder.layers[1].mlp.linear_fc2.weight.grad
    else:
        assert losses == []
        g, gr = model.decoder.layers[0].mlp.linear_fc2.weight.grad, ref.decoder.layers[0].mlp.linear_fc2.weight.grad
    assert torch.allclose(g, gr, atol=1e-5), (g - gr).abs().max()
    return True


def test_1f1b_streaming_two_stages():
    for n_mb in (1, 3, 5):
        assert all(run_distributed(_pp_worker, 2, n_mb))


def _pp_trainer_worker(rank, world, tied):
    """Pipeline-parallel trainer (pp=2): log-probs, loss metrics and parameter gradients equal the single-rank trainer."""
    import dataclasses

    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.parallel.state import ParallelDims, init_parallel_state
    from relax_b200.train.actor import TrainActor, TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    mcfg = dataclasses.replace(get_config("tiny"), tie_word_embeddings=tied)
    ps = init_parallel_state(ParallelDims(pp=2))
    tcfg = TrainConfig(pad_multiple=1, max_tokens_per_gpu=48, global_batch_size=4, n_samples_per_prompt=2,
                       loss=LossConfig(use_kl_loss=False), optim=OptimizerConfig(lr=1e-2, clip_grad=0.0))
    actor = TrainActor(mcfg, tcfg, ps, seed=5)
    g = torch.Generator().manual_seed(1)
    toks = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (20, 17, 23, 19)]
    batch = {"tokens": toks, "response_lengths": [8, 6, 9, 7], "loss_masks": [[1.0] * r for r in (8, 6, 9, 7)],
             "rewards": [1.0, -1.0, 0.5, -0.5]}
    lps = actor.compute_log_prob(batch)["log_probs"]
    grads = {}
    step = actor.optimizer.step

    def recording_step(*a, **k):       # the accumulated gradients as the optimizer sees them
        grads.update({n: p.main_grad.detach().numpy().copy() for n, p in actor.model.named_parameters()})
        return step(*a, **k)

    actor.optimizer.step = recording_step
    m = actor.train(0, dict(batch))
    names = [n for n, _ in actor.model.named_parameters()]
    return [x.detach().numpy().copy() for x in lps], {k: float(v) for k, v in m.items() if k != "train_time"}, names, grads


import pytest


@pytest.mark.parametrize("tied", [False, True])
def test_pipeline_parallel_trainer_matches_single_rank(tied):
    import dataclasses

    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.train.actor import TrainActor, TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    out = run_distributed(_pp_trainer_worker, 2, tied, timeout=600)
    mcfg = dataclasses.replace(get_config("tiny"), tie_word_embeddings=tied)
    tcfg = TrainConfig(pad_multiple=1, max_tokens_per_gpu=48, global_batch_size=4, n_samples_per_prompt=2,
                       loss=LossConfig(use_kl_loss=False), optim=OptimizerConfig(lr=1e-2, clip_grad=0.0))
    ref = TrainActor(mcfg, tcfg, seed=5)
    g = torch.Generator().manual_seed(1)
    toks = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (20, 17, 23, 19)]
    batch = {"tokens": toks, "response_lengths": [8, 6, 9, 7], "loss_masks": [[1.0] * r for r in (8, 6, 9, 7)],
             "rewards": [1.0, -1.0, 0.5, -0.5]}
    lps = ref.compute_log_prob(batch)["log_probs"]
    ref_params = {}
    step = ref.optimizer.step

    def recording_step(*a, **k):
        ref_params.update({n: p.main_grad.detach().clone() for n, p in ref.model.named_parameters()})
        return step(*a, **k)

    ref.optimizer.step = recording_step
    m = ref.train(0, dict(batch))
    for rank in range(2):
        got_lp, got_m, names, after = out[rank]
        for a, b in zip(got_lp, lps):                      # every stage returns the log-probs
            assert torch.allclose(torch.from_numpy(a), b.detach(), atol=1e-5)
        for k in ("loss", "pg_loss"):
            if k in m:
                assert abs(got_m[k] - float(m[k])) < 1e-5, (k, got_m[k], m[k])
        assert abs(got_m["grad_norm"] - m["grad_norm"]) < 1e-4
    # stage 0 holds layer 0 (local name layers.0), stage 1 holds layer 1 (local name layers.0 as well)
    a0, a1 = ({k: torch.from_numpy(v) for k, v in out[r][3].items()} for r in range(2))
    assert torch.allclose(a0["decoder.layers.0.mlp.linear_fc2.weight"], ref_params["decoder.layers.0.mlp.linear_fc2.weight"], atol=1e-6)
    assert torch.allclose(a1["decoder.layers.0.mlp.linear_fc2.weight"], ref_params["decoder.layers.1.mlp.linear_fc2.weight"], atol=1e-5)
    assert torch.allclose(a0["embedding.word_embeddings.weight"], ref_params["embedding.word_embeddings.weight"], atol=1e-5)
    if tied:
        assert torch.allclose(a1["embedding.word_embeddings.weight"], ref_params["embedding.word_embeddings.weight"], atol=1e-5)
