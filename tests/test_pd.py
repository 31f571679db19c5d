"""Prefill / decode disaggregation between two engines: same tokens and log-probs as one engine, KV rows re-blocked
for the decode engine's own block size, back-pressure when the decode cache is full, and the hand-over across ranks."""
import pytest
import torch

from relax_b200.models.config import get_config
from relax_b200.models.transformer import GPTModel
from relax_b200.parallel.state import single_process_state
from relax_b200.rollout.engine import RolloutEngine, SamplingParams
from relax_b200.rollout.pd import PDEngine, PeerTransfer, attach, can_attach, detach
from relax_b200.weight_sync.plan import TrainerLayout
from relax_b200.weight_sync.sync import WeightSync
from tests._mp import run_distributed


def _engine(cfg, params, **kw):
    import torch.distributed as dist

    me = dist.get_rank() if dist.is_initialized() else 0
    e = RolloutEngine(cfg, device="cpu", dtype=torch.float32, **kw)
    WeightSync(cfg, TrainerLayout(tp=1), 1, [me], [me]).update_weights(params, e.weights, e, version=3)
    return e


def _setup():
    cfg = get_config("tiny")
    params = {k: v.detach() for k, v in GPTModel(cfg, single_process_state(), seed=11).named_parameters()}
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (4, 9, 17, 30, 12)]
    prompts.append(list(prompts[2]))
    return cfg, params, prompts, [0, 1, 2, 3, 4, 2]


def test_pd_pair_matches_one_engine_and_reblocks_the_cache():
    cfg, params, prompts, keys = _setup()
    one = _engine(cfg, params, num_kv_blocks=128, block_size=8)
    pd = PDEngine(_engine(cfg, params, num_kv_blocks=64, block_size=16), _engine(cfg, params, num_kv_blocks=256, block_size=4))
    sp = SamplingParams(temperature=0.0, max_new_tokens=10)
    want = one.generate(prompts, sp, group_keys=keys)
    got = pd.generate(prompts, sp, group_keys=keys)
    for a, b in zip(want, got):
        assert a.output == b.output and b.finish_reason == a.finish_reason and b.weight_versions == [3] * 10
        assert torch.allclose(torch.tensor(a.logprobs), torch.tensor(b.logprobs), atol=1e-5)
    assert pd.stats["handed_over"] == 6 and pd.stats["kv_bytes"] == sum(len(p) for p in prompts) * cfg.num_layers * 2 * cfg.kv_size * 4
    assert not pd.prefill.running and pd.prefill.bm.num_free == pd.prefill.bm.num_blocks       # the prefill side holds nothing
    assert pd.decode.bm.num_free == pd.decode.bm.num_blocks
    # requests that end with their first token never travel
    short = pd.generate(prompts[:2], SamplingParams(temperature=0.0, max_new_tokens=1))
    assert [r.output for r in short] == [w.output[:1] for w in want[:2]] and pd.stats["handed_over"] == 6


def test_prefilled_requests_wait_for_room_on_the_decode_engine():
    cfg, params, prompts, keys = _setup()
    one = _engine(cfg, params, num_kv_blocks=128, block_size=8)
    sp = SamplingParams(temperature=0.0, max_new_tokens=6)
    want = one.generate(prompts, sp)
    # the decode cache holds about two requests at a time
    pd = PDEngine(_engine(cfg, params, num_kv_blocks=64, block_size=8), _engine(cfg, params, num_kv_blocks=11, block_size=8))
    got = pd.generate(prompts, sp)
    assert [r.output for r in got] == [r.output for r in want]
    assert pd.stats["decode_steps"] >= 5 * 2         # at least two waves of five decode steps
    tiny = PDEngine(_engine(cfg, params, num_kv_blocks=64, block_size=8), _engine(cfg, params, num_kv_blocks=3, block_size=8))
    with pytest.raises(RuntimeError, match="too small"):
        tiny.generate(prompts[3:4], sp)


def test_detach_attach_by_hand_with_sampling():
    """A request sampled with temperature continues on the other engine with its own parameters and random stream."""
    cfg, params, prompts, _ = _setup()
    a, b = _engine(cfg, params, num_kv_blocks=64, block_size=8), _engine(cfg, params, num_kv_blocks=64, block_size=8)
    a.add_request(prompts[1], SamplingParams(temperature=0.8, top_p=0.9, max_new_tokens=7))
    a.step()
    (item,) = detach(a, list(a.running))
    assert item.kv.shape == (cfg.num_layers, 2, len(prompts[1]), cfg.num_query_groups, cfg.head_dim) and len(item.output) == 1
    assert can_attach(b, item)
    r = attach(b, item)
    while b.running:
        b.step()
    assert len(r.output) == 7 and len(r.logprobs) == 7 and r.finish_reason == "length" and r.output[0] == item.output[0]


def _peer_worker(rank, world):
    cfg, params, prompts, keys = _setup()
    sp = SamplingParams(temperature=0.0, max_new_tokens=5)
    wire = PeerTransfer(0, 1)
    if rank == 0:
        eng = _engine(cfg, params, num_kv_blocks=64, block_size=8)
        for p in prompts[:3]:
            eng.add_request(p, sp)
        eng.step()
        wire.send(detach(eng, list(eng.running)))
        return None
    eng = _engine(cfg, params, num_kv_blocks=64, block_size=4)
    reqs = [attach(eng, it) for it in wire.recv()]
    while eng.running:
        eng.step()
    ref = _engine(cfg, params, num_kv_blocks=64, block_size=8).generate(prompts[:3], sp)
    return [r.output for r in reqs] == [r.output for r in ref]


def test_hand_over_between_ranks():
    out = run_distributed(_peer_worker, 2, timeout=300)
    assert out[1] is True
