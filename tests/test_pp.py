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
