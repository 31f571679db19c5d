import torch

from relax_b200.models.config import get_config
from relax_b200.rollout.engine import BlockManager, RolloutEngine, SamplingParams
from relax_b200.train.actor import TrainActor, TrainConfig
from relax_b200.weight_sync.plan import TrainerLayout
from relax_b200.weight_sync.sync import WeightSync


def _pair(kv_blocks=256, **kw):
    cfg = get_config("tiny")
    actor = TrainActor(cfg, TrainConfig(), seed=0, with_optimizer=False)
    eng = RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=kv_blocks, block_size=8, **kw)
    WeightSync(cfg, TrainerLayout(), 1, [0], [0]).update_weights(dict(actor.named_local_params()), eng.weights, eng, 1)
    return cfg, actor, eng


def test_block_manager_refcounts():
    bm = BlockManager(4, 8)
    a, b = bm.alloc(), bm.alloc()
    bm.share(a)
    bm.release([a])
    assert bm.num_free == 2
    bm.release([a, b])
    assert bm.num_free == 4 and bm.blocks_for(17) == 3


def test_rollout_logprobs_match_trainer_forward():
    cfg, actor, eng = _pair()
    torch.manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (5, 11, 8)]
    res = eng.generate(prompts, SamplingParams(max_new_tokens=9))
    assert eng.weight_version == 1
    batch = {"tokens": [r.prompt + r.output for r in res], "response_lengths": [len(r.output) for r in res]}
    lp = actor.compute_log_prob(batch)["log_probs"]
    for r, l in zip(res, lp):
        assert len(r.output) == 9 and r.finish_reason == "length"
        assert torch.allclose(torch.tensor(r.logprobs), l, atol=1e-4)
    assert eng.bm.num_free == eng.bm.num_blocks       # every block returned


def test_group_prefix_sharing_equals_independent_prefill():
    cfg, actor, eng = _pair()
    prompt = list(range(3, 22))                        # 19 tokens: 2 full blocks + partial tail
    sp = SamplingParams(max_new_tokens=6)
    shared = eng.generate([prompt] * 4, sp, group_keys=[0] * 4)
    assert eng.stats["prefill_tokens"] == len(prompt)  # one prefill for the whole group
    # log-probs of every member agree with a fresh trainer forward (KV sharing is exact)
    batch = {"tokens": [r.prompt + r.output for r in shared], "response_lengths": [6] * 4}
    for r, l in zip(shared, actor.compute_log_prob(batch)["log_probs"]):
        assert torch.allclose(torch.tensor(r.logprobs), l, atol=1e-4)
    assert len({tuple(r.output) for r in shared}) > 1  # members sample independently
    assert eng.bm.num_free == eng.bm.num_blocks


def test_continuous_batching_under_kv_pressure_and_eos():
    cfg, actor, eng = _pair(kv_blocks=12, max_running=8)   # 96 KV slots: at most ~3 requests of 8+20 tokens
    eng.eos = 7
    prompts = [[i + 1] * 8 for i in range(6)]
    res = eng.generate(prompts, SamplingParams(max_new_tokens=20))
    assert len(res) == 6 and all(r.status == "finished" for r in res)
    for r in res:
        assert r.finish_reason in ("stop", "length")
        if r.finish_reason == "stop":
            assert r.output[-1] == 7
    assert eng.bm.num_free == 12


def test_abort_returns_partial_and_resume_continues():
    cfg, actor, eng = _pair()
    rid = eng.add_request([1, 2, 3, 4], SamplingParams(max_new_tokens=10))
    for _ in range(4):
        eng.step()
    part = eng.abort_all()
    assert len(part) == 1 and part[0].status == "aborted" and 0 < len(part[0].output) < 10
    assert eng.bm.num_free == eng.bm.num_blocks
    got = len(part[0].output)
    eng.add_request(part[0].prompt, SamplingParams(max_new_tokens=10), resume_output=part[0].output,
                    resume_logprobs=part[0].logprobs)
    done = []
    while eng.has_work:
        done += eng.step()
    assert len(done[0].output) == 10 and done[0].output[:got] == part[0].output


def test_pause_and_memory_release():
    cfg, actor, eng = _pair()
    eng.add_request([1, 2, 3], SamplingParams(max_new_tokens=2))
    eng.pause_generation()
    assert eng.step() == [] and eng.has_work
    eng.continue_generation()
    while eng.has_work:
        eng.step()
    eng.release_memory_occupation(("kv_cache", "weights"))
    assert eng.kv is None and eng.weights.flat is None
    eng.resume_memory_occupation(("kv_cache", "weights"))
    assert eng.kv is not None and eng.weights.flat is not None


def test_memory_saver_keeps_views_across_pause_resume():
    """CPU emulation of the pausable buffers: release/resume keeps the tensor objects and generation still works."""
    import torch
    from relax_b200.models.config import get_config
    from relax_b200.rollout.engine import RolloutEngine, SamplingParams

    cfg = get_config("tiny")
    eng = RolloutEngine(cfg, device="cpu", num_kv_blocks=32, block_size=4, memory_saver=True)
    eng.weights.flat.normal_(0, 0.02)
    w0 = eng.weights.flat.clone()
    kv_obj, p_obj = eng.kv, eng.weights.p["embed"]
    sp = SamplingParams(temperature=1.0, max_new_tokens=4)
    out0 = eng.generate([[1, 2, 3]], sp)[0].output
    eng.release_memory_occupation(("kv_cache", "cuda_graph", "weights"))
    assert eng._kv_buf.paused and eng.weights._buf.paused
    eng.resume_memory_occupation(("kv_cache", "weights"))
    assert eng.kv is kv_obj and eng.weights.p["embed"] is p_obj
    assert float(eng.weights.flat.abs().sum()) == 0.0     # contents are not preserved
    eng.weights.flat.copy_(w0)
    assert len(eng.generate([[1, 2, 3]], sp)[0].output) == len(out0)


def test_windowed_decode_equals_host_driven_loop():
    """Several decode steps per host round trip (batch state advanced by ``decode_advance``) give the same tokens,
    log-probs and finish reasons as one host round trip per step, for fixed-length and for EOS-terminated requests,
    under KV pressure (requests admitted while others run) and with a group sharing its prompt blocks."""
    outs = []
    for windowed in (False, True):
        cfg, actor, eng = _pair(kv_blocks=64, max_running=8, windowed_decode=windowed, decode_window=5)
        torch.manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (5, 11, 8, 3)]
        fixed = eng.generate(prompts, SamplingParams(max_new_tokens=13, ignore_eos=True))
        grp = eng.generate([list(range(3, 22))] * 3, SamplingParams(max_new_tokens=7, ignore_eos=True), group_keys=[0] * 3)
        assert eng.bm.num_free == eng.bm.num_blocks - (1 if windowed else 0)     # the scratch block of padding rows
        outs.append([(r.output, r.logprobs, r.finish_reason) for r in fixed + grp])
        if windowed:
            assert eng.stats["graph_replays"] >= 13 + 7 - 2
    for (o0, l0, f0), (o1, l1, f1) in zip(*outs):
        assert o0 == o1 and f0 == f1 == "length"
        assert torch.allclose(torch.tensor(l0), torch.tensor(l1), atol=1e-6)
    # EOS inside a window: the row stops on the device too, later ring entries are ignored, blocks come back
    cfg, actor, eng = _pair(kv_blocks=24, max_running=4, windowed_decode=True, decode_window=6)
    eng.eos = 7
    res = eng.generate([[i + 1] * 8 for i in range(6)], SamplingParams(max_new_tokens=20, stop_token_ids=(9,)))
    assert len(res) == 6 and all(r.status == "finished" for r in res)
    for r in res:
        assert r.finish_reason in ("stop", "length") and len(r.output) <= 20
        if r.finish_reason == "stop":
            assert r.output[-1] in (7, 9) and not any(t in (7, 9) for t in r.output[:-1])
        else:
            assert not any(t in (7, 9) for t in r.output)
    assert eng.bm.num_free == eng.bm.num_blocks - 1
    batch = {"tokens": [r.prompt + r.output for r in res], "response_lengths": [len(r.output) for r in res]}
    for r, l in zip(res, actor.compute_log_prob(batch)["log_probs"]):
        assert torch.allclose(torch.tensor(r.logprobs), l, atol=1e-4)


def test_moe_engine_logprobs_match_trainer_forward():
    """A mixture-of-experts model in the rollout engine (grouped expert path, rows of foreign experts parked) returns
    the log-probs the trainer computes for the same tokens."""
    cfg = get_config("tiny-moe")
    actor = TrainActor(cfg, TrainConfig(), seed=0, with_optimizer=False)
    eng = RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=128, block_size=8)
    WeightSync(cfg, TrainerLayout(), 1, [0], [0]).update_weights(dict(actor.named_local_params()), eng.weights, eng, 1)
    torch.manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (6, 9)]
    res = eng.generate(prompts, SamplingParams(max_new_tokens=7))
    batch = {"tokens": [r.prompt + r.output for r in res], "response_lengths": [len(r.output) for r in res]}
    for r, l in zip(res, actor.compute_log_prob(batch)["log_probs"]):
        assert torch.allclose(torch.tensor(r.logprobs), l, atol=1e-4)
