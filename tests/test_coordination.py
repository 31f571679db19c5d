"""Role barriers, inference permits, user-code loaders and the small agreement collectives (CPU)."""
import asyncio
import threading
import time

import pytest
import torch

from relax_b200.orchestration.coordination import BarrierTimeout, PeerStepBarrier, RolloutOffloadBarrier
from relax_b200.rollout import custom_generate as CG
from relax_b200.rollout.request_permit import GenerationAborted, InferencePermitManager, benchmark, capacity_for
from tests._mp import run_distributed


def test_offload_and_peer_barriers():
    state = {"s": "onload", "actor": 3, "ref": 4}
    threading.Timer(0.15, lambda: state.update(s="offload")).start()
    waited = RolloutOffloadBarrier(lambda: state["s"], 0.01).wait_offloaded(5)
    assert 0.1 < waited < 2
    state["s"] = "onload"
    with pytest.raises(BarrierTimeout):
        RolloutOffloadBarrier(lambda: state["s"], 0.01).wait_offloaded(0.1)
    b = PeerStepBarrier({"actor": lambda: state["actor"], "ref": lambda: state["ref"]}, 0.01)
    assert b.list_pending(3) == [("actor", 3)] and not b.is_empty()
    threading.Timer(0.1, lambda: state.update(actor=4)).start()
    assert b.wait_completed_round(3, 5) >= 1
    with pytest.raises(BarrierTimeout):
        b.wait_completed_round(4, 0.1)         # a peer that never advances surfaces as an error, not a hang
    assert PeerStepBarrier({}).wait_completed_round(100) == 0


def test_permits_bound_concurrency_and_abort():
    assert capacity_for(16, 8, 2) == 64
    with pytest.raises(ValueError):
        capacity_for(1, 1, 4)
    m = InferencePermitManager(2)
    live, peak = [0], [0]

    def work():
        with m.permit():
            live[0] += 1
            peak[0] = max(peak[0], live[0])
            time.sleep(0.02)
            live[0] -= 1

    ths = [threading.Thread(target=work) for _ in range(8)]
    [t.start() for t in ths]
    [t.join() for t in ths]
    assert peak[0] == 2 and m.peak == 2 and m.granted == 8 and m.in_use == 0
    # abort while waiting, abort right after the grant, timeout
    m.acquire(); m.acquire()
    flag = {"abort": False}
    threading.Timer(0.1, lambda: flag.update(abort=True)).start()
    with pytest.raises(GenerationAborted):
        m.acquire(lambda: flag["abort"])
    with pytest.raises(TimeoutError):
        m.acquire(timeout_s=0.1)
    m.release()
    with pytest.raises(GenerationAborted):
        m.acquire(lambda: True)
    assert m.in_use == 1                 # the aborted grant was handed back
    m.resize(3)
    m.acquire(timeout_s=1); m.acquire(timeout_s=1)
    assert m.in_use == 3
    for _ in range(3):
        m.release()
    with pytest.raises(RuntimeError):
        m.release()


def test_async_permits_and_benchmark_shape():
    m = InferencePermitManager(3)

    async def go():
        async def one():
            async with m.apermit():
                await asyncio.sleep(0.01)
        await asyncio.gather(*[one() for _ in range(12)])

    asyncio.run(go())
    assert m.granted == 12 and m.peak <= 3 and m.in_use == 0
    fast = benchmark(sessions=24, turns=2, capacity=4, model_ms=3, tool_ms=6)
    slow = benchmark(sessions=24, turns=2, capacity=4, model_ms=3, tool_ms=6, hold_over_tools=True)
    assert fast["peak_in_flight"] <= 4 and fast["granted"] == 48
    assert fast["seconds"] < slow["seconds"]          # tool time overlaps other sessions' requests


def test_load_user_functions(tmp_path):
    f = tmp_path / "user_gen.py"
    f.write_text("def gen(engine, samples, params):\n    return samples\n\n"
                 "def bad(x):\n    return x\n\nclass K:\n    @staticmethod\n    def rm(sample):\n        return 1.0\n\n"
                 "gen.manages_inference_permit = True\n")
    g = CG.load_generate_function(f"{f}:gen", default=None)
    assert g(None, [1], None) == [1] and CG.manages_inference_permit(g)
    assert CG.load_generate_function(None, default=len) is len
    with pytest.raises(TypeError):
        CG.load_function(f"{f}:bad", 3)
    assert CG.load_function(f"{f}:K.rm", 1)(None) == 1.0
    assert CG.load_object("math:pi") > 3 and CG.load_object("os.path.join") is __import__("os").path.join
    with pytest.raises(AttributeError):
        CG.load_object(f"{f}:nope")
    with pytest.raises(FileNotFoundError):
        CG.load_object(str(tmp_path / "missing.py") + ":x")
    with pytest.raises(ValueError):
        CG.load_object("justaname")


def _coll_worker(rank, world):
    from relax_b200.parallel.collective_utils import ConditionalBranchSync, agree_drained, chunked_all_reduce
    from relax_b200.parallel.state import ParallelDims, init_parallel_state

    ps = init_parallel_state(ParallelDims(tp=2))
    out = {"drain_mixed": agree_drained(rank == 0, [ps.tp]), "drain_all": agree_drained(True, [ps.tp, ps.pp])}
    w = torch.nn.Parameter(torch.ones(3))
    sync = ConditionalBranchSync(ps.tp)
    y = sync.run(rank == 0, lambda: (w * 2).sum(), lambda: w.sum())
    y.backward()
    out["y"], out["grad"], out["dummy"] = float(y), w.grad.clone(), sync.dummy_runs
    out["none"] = sync.run(False, lambda: 1, lambda: 2)
    flat = torch.arange(10, dtype=torch.float32) * (rank + 1)
    out["calls"] = chunked_all_reduce(flat, ps.tp, chunk_bytes=16)
    out["flat"] = flat
    return out


def test_agreement_collectives_two_ranks():
    o0, o1 = run_distributed(_coll_worker, 2)
    assert o0["drain_mixed"] is False and o1["drain_mixed"] is False and o0["drain_all"] and o1["drain_all"]
    assert o0["y"] == 6.0 and o1["y"] == 0.0 and o1["dummy"] == 1 and o0["dummy"] == 0
    assert torch.equal(o1["grad"], torch.zeros(3)) and torch.equal(o0["grad"], torch.full((3,), 2.0))
    assert o0["none"] is None and o1["none"] is None
    assert o0["calls"] == 3 and torch.equal(o0["flat"], torch.arange(10, dtype=torch.float32) * 3) and torch.equal(o0["flat"], o1["flat"])


def test_chat_endpoint_takes_a_permit_and_honours_abort():
    from relax_b200.rollout.agentic import Tokenizer
    from relax_b200.rollout.openai_api import ChatService

    tok = Tokenizer(encode=lambda s: [ord(c) for c in s], decode=lambda t: "".join(chr(97 + x % 26) for x in t))
    m = InferencePermitManager(1)
    gen = lambda prompts, n, keys: [([5, 6, 7], [-0.1, -0.2, -0.3], "stop", [0]) for _ in prompts]
    flag = {"abort": False}
    svc = ChatService(gen, tok, permits=m, abort_check=lambda: flag["abort"])
    r = svc.chat({"messages": [{"role": "user", "content": "hi"}]})
    assert r["choices"][0]["message"]["content"] and m.granted == 1 and m.in_use == 0
    flag["abort"] = True
    with pytest.raises(GenerationAborted):
        svc.chat({"messages": [{"role": "user", "content": "hi"}]})
    assert m.in_use == 0


def test_custom_generate_and_reward_paths_drive_the_colocated_loop(tmp_path):
    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.orchestration.colocate import ColocateConfig, ColocatedGRPO
    from relax_b200.train.actor import TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    f = tmp_path / "user_code.py"
    f.write_text(
        "from relax_b200.types import SampleStatus\n"
        "CALLS = []\n"
        "def generate(engine, samples, sp):\n"
        "    res = engine.generate([s.tokens for s in samples], sp, group_keys=[s.group_index for s in samples])\n"
        "    for s, r in zip(samples, res):\n"
        "        s.tokens = list(r.prompt) + list(r.output)\n"
        "        s.response_length = len(r.output)\n"
        "        s.rollout_log_probs = list(r.logprobs)\n"
        "        s.status = SampleStatus.COMPLETED\n"
        "        s.metadata['custom'] = True\n"
        "    CALLS.append(len(samples))\n"
        "    return samples\n"
        "def reward(sample):\n"
        "    return float(sum(sample.tokens[-sample.response_length:]) % 3 == 0)\n")
    cfg = ColocateConfig(model=get_config("tiny"), train=TrainConfig(global_batch_size=4, n_samples_per_prompt=2, pad_multiple=1,
                         max_tokens_per_gpu=256, loss=LossConfig(), optim=OptimizerConfig(lr=1e-4)),
                         rollout_batch_size=2, prompt_len=8, max_response_len=8, kv_blocks=64, num_prompts=16,
                         custom_generate_function_path=f"{f}:generate", custom_rm_path=f"{f}:reward")
    run = ColocatedGRPO(cfg)
    m = run.step()
    assert CG.load_object(f"{f}:CALLS") == [4] and 0.0 <= m["raw_reward_mean"] <= 1.0


def test_dynamic_sampling_filter_in_the_colocated_loop():
    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.orchestration.colocate import ColocateConfig, ColocatedGRPO
    from relax_b200.train.actor import TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    cfg = ColocateConfig(model=get_config("tiny"), train=TrainConfig(global_batch_size=8, n_samples_per_prompt=4, pad_multiple=1,
                         max_tokens_per_gpu=512, loss=LossConfig(), optim=OptimizerConfig(lr=1e-4)),
                         rollout_batch_size=2, prompt_len=8, max_response_len=8, kv_blocks=128, num_prompts=64, rm_type="token_sum_parity",
                         dynamic_sampling_filter_path="relax_b200.rollout.filters:check_reward_nonzero_std", over_sampling_batch_size=4,
                         offload_rollout=False)
    run = ColocatedGRPO(cfg)
    m = run.step()
    assert m["rollout/dynamic_sampling/generated_groups"] >= 4 and m["rollout/dynamic_sampling/rounds"] >= 1
    # every kept group has mixed rewards, so no group is wasted on a zero advantage
    samples = run.generate(1)
    by_group = {}
    for s in samples:
        by_group.setdefault(s.group_index, []).append(s.reward)
    assert len(by_group) == 2 and all(len(set(v)) > 1 for v in by_group.values())


def test_reward_postprocess_sample_filter_and_rollout_postprocess_hooks(tmp_path):
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    f = tmp_path / "hooks.py"
    f.write_text(
        "import torch\n"
        "LOG = []\n"
        "def post(samples):\n"
        "    raw = torch.tensor([float(s.reward) for s in samples])\n"
        "    LOG.append(('post', len(samples)))\n"
        "    return raw, raw * 2 - 1\n"
        "def drop_first(cfg, samples):\n"
        "    samples[0].remove_sample = True\n"
        "    LOG.append(('filter', len(samples)))\n"
        "def tag(cfg, samples):\n"
        "    for s in samples:\n"
        "        s.metadata['tagged'] = True\n"
        "    LOG.append(('tag', len(samples)))\n"
        "    return samples\n")
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "8", "--rm-type", "token_sum_parity",
                    "--custom-reward-post-process-path", f"{f}:post", "--rollout-sample-filter-path", f"{f}:drop_first",
                    "--rollout-data-postprocess-path", f"{f}:tag"])
    c = Controller(a, device="cpu")
    m = c.runner.step()
    assert [k for k, _ in CG.load_object(f"{f}:LOG")] == ["filter", "tag", "post"]
    assert 0.0 <= m["raw_reward_mean"] <= 1.0
