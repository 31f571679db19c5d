"""Agentic multi-turn rollout, session forest, OpenAI-compatible endpoint, generative reward model."""
import json
import urllib.request

import pytest

from relax_b200.rewards.genrm import GenRM, JudgeEngine, parse_verdict
from relax_b200.rollout import agentic as A
from relax_b200.rollout.openai_api import ChatService, serve

TOK = A.Tokenizer(encode=lambda s: [ord(c) for c in s], decode=lambda t: "".join(chr(x) for x in t))


class _CountEnv:
    """The agent must say 'ping' twice; each tool reply is 'pong'."""

    def __init__(self):
        self.n = 0

    def reset(self):
        return [{"role": "user", "content": "play"}]

    def step(self, text):
        self.n += 1
        ok = "ping" in text
        return ("pong", 1.0 if ok else 0.0, self.n >= 2)


def _fake_generate(prompts, max_new, keys):
    return [(TOK.encode("ping")[:max_new], [-0.1] * min(4, max_new), "stop", [3]) for _ in prompts]


def test_episode_masks_and_logprobs():
    s = A.run_episode(_CountEnv(), _fake_generate, TOK, max_turns=5)
    smp = s.to_sample(group_index=0, index=0)
    text = TOK.decode(smp.tokens)
    assert text.count("ping") == 2 and text.count("pong") == 1 and s.reward == 2.0 and s.turns == 2
    assert len(smp.loss_mask) == smp.response_length == len(smp.rollout_log_probs)
    gen = [t for t, m in zip(smp.tokens[-smp.response_length:], smp.loss_mask) if m]
    assert TOK.decode(gen) == "pingping"
    assert all((lp == -0.1) == bool(m) for lp, m in zip(smp.rollout_log_probs, smp.loss_mask))
    assert smp.weight_versions == [3]


def test_lockstep_batching_admission_and_truncation():
    calls = []

    def gen(prompts, max_new, keys):
        calls.append(len(prompts))
        return _fake_generate(prompts, max_new, keys)

    sess = A.run_episodes([_CountEnv() for _ in range(5)], gen, TOK, max_concurrent=2)
    assert all(s.done and s.turns == 2 for s in sess) and max(calls) == 2
    short = A.run_episode(_CountEnv(), _fake_generate, TOK, max_context=30)
    assert short.truncated and len(short.tokens) <= 30


def test_session_forest_fork_shares_prefix():
    f = A.SessionForest()
    a = f.new()
    a.append([1, 2, 3, 4], 0)
    a.prompt_len = 4
    a.append([5, 6], 1, [-1.0, -2.0])
    b = f.fork(a.sid, at_tokens=5)
    b.append([9], 1, [-3.0])
    assert f.shared_prefix(a.sid, b.sid) == 5 and f.children(a.sid) == [b.sid] and b.branch_point == 5
    assert b.to_sample().rollout_log_probs == [-1.0, -3.0]


def test_env_registry():
    A.register_env("count")(_CountEnv)
    assert isinstance(A.make_env("count"), _CountEnv)
    with pytest.raises(KeyError):
        A.make_env("nope")


def test_openai_endpoint_roundtrip_and_session_sample():
    svc = ChatService(_fake_generate, TOK)
    srv, url = serve(svc)
    try:
        def post(body, sid):
            req = urllib.request.Request(url + "/v1/chat/completions", data=json.dumps(body).encode(),
                                         headers={"Content-Type": "application/json", "X-Session-Id": sid})
            return json.loads(urllib.request.urlopen(req, timeout=10).read())

        msgs = [{"role": "user", "content": "hi"}]
        r1 = post({"messages": msgs, "max_tokens": 8, "logprobs": True}, "s1")
        assert r1["choices"][0]["message"]["content"] == "ping" and r1["usage"]["completion_tokens"] == 4
        assert len(r1["choices"][0]["logprobs"]["content"]) == 4
        msgs += [r1["choices"][0]["message"], {"role": "tool", "content": "pong"}]
        post({"messages": msgs, "max_tokens": 8}, "s1")
        smp = svc.finish_session("s1", reward=1.0)
        assert sum(smp.loss_mask) == 8 and smp.reward == 1.0 and "pong" in TOK.decode(smp.tokens)
        models = json.loads(urllib.request.urlopen(url + "/v1/models", timeout=10).read())
        assert models["data"][0]["id"] == svc.model_name
        # the short forms of the routes, and the state page
        assert json.loads(urllib.request.urlopen(url + "/models", timeout=10).read())["data"][0]["id"] == svc.model_name
        assert json.loads(urllib.request.urlopen(url + "/healthz", timeout=10).read())["ok"] is True
        req = urllib.request.Request(url + "/chat/completions", data=json.dumps({"messages": [{"role": "user", "content": "x"}]}).encode(),
                                     headers={"Content-Type": "application/json", "X-Session-Id": "s2"})
        assert json.loads(urllib.request.urlopen(req, timeout=10).read())["choices"][0]["message"]["content"] == "ping"
        st = json.loads(urllib.request.urlopen(url + "/debug_state", timeout=10).read())
        assert st["session_count"] == 2 and st["open_sessions"] == 1 and st["turns"] == 3
    finally:
        srv.shutdown()


def test_genrm_parsing_failover_and_default():
    assert parse_verdict("blah Verdict: correct") == 1.0 and parse_verdict("Verdict: wrong") == 0.0
    assert parse_verdict("Score: 7") == 0.7 and parse_verdict("score - 3/4") == 0.75 and parse_verdict("??", 0.5) == 0.5

    def broken(prompts, n):
        raise RuntimeError("engine lost")

    good = JudgeEngine(lambda prompts, n: ["Verdict: correct" if "42" in p.split("Candidate answer:")[1] else "Verdict: incorrect" for p in prompts])
    rm = GenRM([JudgeEngine(broken), good])
    assert rm.score(["q", "q"], ["42", "42"], ["it is 42", "it is 41"]) == [1.0, 0.0]
    assert rm.failures == 1 and not rm.engines[0].healthy
    rm.recover(lambda e: True)
    assert rm.engines[0].healthy
    dead = GenRM([JudgeEngine(broken)], default=0.25)
    assert dead.score(["q"], ["r"], ["a"]) == [0.25]


def test_ifbench_remote_and_dapo_genrm_rewards():
    import json
    import threading
    from http.server import BaseHTTPRequestHandler, HTTPServer

    from relax_b200.rewards import get_reward_spec
    from relax_b200.rewards.rules import make_dapo_genrm_reward, remote_rm_reward
    from relax_b200.types import Sample

    s = Sample(prompt="p", response="<think>x</think>one two three four. done", label={"min_words": 4, "forbidden_words": ["five"],
                                                                                       "ends_with": "done", "bogus": 1})
    assert get_reward_spec("ifbench").fn(s) == 0.75
    s.label = json.dumps({"max_words": 2})
    assert get_reward_spec("ifbench").fn(s) == 0.0

    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            out = json.dumps({"reward": 1.0 if body["label"] in body["response"] else 0.0}).encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(out)))
            self.end_headers()
            self.wfile.write(out)

    srv = HTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        url = f"http://127.0.0.1:{srv.server_address[1]}"
        assert remote_rm_reward(Sample(prompt="q", response="the answer is 42", label="42"), url=url) == 1.0
        assert remote_rm_reward(Sample(prompt="q", response="no idea", label="42"), url=url) == 0.0
    finally:
        srv.shutdown()

    rm = GenRM([JudgeEngine(lambda prompts, n: ["Verdict: correct"] * len(prompts))])
    fn = make_dapo_genrm_reward(rm)
    assert fn(Sample(prompt="q", response="Answer: 7", label="7"))["score"] == 1.0          # rule decides
    assert fn(Sample(prompt="q", response="Answer: 8", label="7"))["score"] == -1.0
    assert fn(Sample(prompt="q", response="it is seven", label="7"))["pred"] == "[GENRM]"   # judge decides


def test_env_generate_plugs_into_the_colocated_loop(tmp_path):
    import json

    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    @A.register_env("echo_once")
    class EchoOnce:
        def __init__(self, bonus=0.0):
            self.bonus, self.n = bonus, 0

        def reset(self):
            return [{"role": "user", "content": "say something"}]

        def step(self, text):
            self.n += 1
            return ("tool says hi", 0.0, False) if self.n == 1 else (None, 1.0 + self.bonus, True)

    f = tmp_path / "prompts.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": "unused", "label": None, "metadata": {"env": {"name": "echo_once", "bonus": 0.5 * i}, "max_turns": 3}})
                           for i in range(2)) + "\n")
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "6", "--rollout-max-prompt-len", "256", "--prompt-data", str(f),
                    "--input-key", "prompt", "--custom-generate-function-path", "relax_b200.rollout.agentic:env_generate",
                    "--disable-rewards-normalization"])
    c = Controller(a, device="cpu")
    samples = c.runner.generate(0)
    assert len(samples) == 4 and all(s.metadata["turns"] == 2 for s in samples)
    assert sorted({s.reward for s in samples}) == [1.0, 1.5]
    s = samples[0]
    assert len(s.loss_mask) == s.response_length == len(s.rollout_log_probs) and 0 < sum(s.loss_mask) < s.response_length
    m = c.runner.step()
    assert m["raw_reward_mean"] == 1.25


def test_admission_controller_leases_fifo_ageing_and_pressure():
    import threading
    import time

    from relax_b200.rollout.admission import AdmissionController, reservation_tokens

    assert reservation_tokens(100, 50) == 150
    ac = AdmissionController(capacity_tokens=100, max_wait_s=0.4)
    a = ac.acquire(60)
    assert a is not None and not a.bypass
    assert ac.acquire(60, timeout_s=0.0) is None                 # does not fit next to the first lease
    order = []

    def waiter(tag, n):
        l = ac.acquire(n)
        order.append((tag, l.bypass))
        time.sleep(0.02)
        ac.release(l)

    t1 = threading.Thread(target=waiter, args=("big", 70))
    t1.start()
    time.sleep(0.05)
    t2 = threading.Thread(target=waiter, args=("small", 10))      # would fit now, but arrived second: stays behind "big"
    t2.start()
    time.sleep(0.05)
    assert order == []
    ac.release(a)
    t1.join(); t2.join()
    assert [t for t, _ in order] == ["big", "small"] and not any(b for _, b in order)
    # ageing: capacity never frees, the waiter is admitted after max_wait_s and the lease says so
    hold = ac.acquire(100)
    t0 = time.monotonic()
    late = ac.acquire(50)
    assert late.bypass and 0.3 < time.monotonic() - t0 < 2.0
    ac.release(hold); ac.release(late)
    # pressure guard: the engines report a full cache, nothing more is admitted next to a running lease
    usage = [0.99]
    ac2 = AdmissionController(1000, pressure_guard=0.9, max_wait_s=5.0, usage_fn=lambda: usage[0])
    first = ac2.acquire(10)
    assert ac2.acquire(10, timeout_s=0.05) is None
    usage[0] = 0.5
    second = ac2.acquire(10, timeout_s=1.0)
    assert second is not None
    m = ac2.metrics()
    assert m["granted"] == 2 and m["reserved"] == 20 and m["cancelled"] == 1
    ac2.release(first); ac2.release(second)


def test_episodes_run_under_admission_control():
    """Episodes join as leases become available and all finish; the reserved peak respects the capacity."""
    from relax_b200.rollout.admission import AdmissionController

    calls = []

    def gen(prompts, max_new, keys):
        calls.append(len(prompts))
        return _fake_generate(prompts, max_new, keys)

    ac = AdmissionController(capacity_tokens=2 * 300, max_wait_s=5.0)
    out = A.run_episodes([_CountEnv() for _ in range(6)], gen, TOK, max_turns=4, max_new_tokens=50, max_context=300, admission=ac)
    assert len(out) == 6 and all(s.done and s.turns == 2 for s in out)
    m = ac.metrics()
    assert max(calls) <= 2 and m["peak_reserved"] <= 600 and m["reserved"] == 0 and m["granted"] == 6


def test_tool_call_and_reasoning_parsers_and_a_tool_using_session():
    from relax_b200.rollout.openai_api import parse_tool_calls, split_reasoning

    text = 'Let me look.\n<tool_call>\n{"name": "search", "arguments": {"q": "b200"}}\n</tool_call><tool_call>{"name": "open", "arguments": "{\\"id\\": 3}"}</tool_call>'
    content, calls = parse_tool_calls(text, "hermes")
    assert content == "Let me look." and [c["function"]["name"] for c in calls] == ["search", "open"]
    assert json.loads(calls[0]["function"]["arguments"]) == {"q": "b200"} and calls[1]["function"]["arguments"] == '{"id": 3}'
    assert parse_tool_calls("<tool_call>{broken</tool_call>", "qwen")[1] == []
    assert parse_tool_calls('{"name": "f", "parameters": {"x": 1}}', "llama3")[1][0]["function"]["arguments"] == '{"x": 1}'
    assert split_reasoning("<think>step 1\nstep 2</think>\n\nThe answer is 4.", "qwen3") == ("step 1\nstep 2", "The answer is 4.")
    assert split_reasoning("<think>cut off while thin", "deepseek-r1") == ("cut off while thin", "")
    assert split_reasoning("no thoughts here", "qwen3") == (None, "no thoughts here")
    with pytest.raises(ValueError):
        parse_tool_calls("x", "nope")

    # a scripted policy: thinks, calls a tool, then answers; the session keeps one token stream through both requests
    script = iter(['<think>need data</think><tool_call>{"name": "lookup", "arguments": {"k": 1}}</tool_call>', "It is 42."])

    def gen(prompts, max_new, keys):
        t = next(script)
        return [(TOK.encode(t), [-0.5] * len(TOK.encode(t)), "stop", [7]) for _ in prompts]

    svc = ChatService(gen, TOK, tool_call_parser="hermes", reasoning_parser="qwen3")
    tools = [{"type": "function", "function": {"name": "lookup", "parameters": {"type": "object"}}}]
    msgs = [{"role": "user", "content": "what is k?"}]
    r1 = svc.chat({"messages": msgs, "tools": tools}, session_key="s")
    m1 = r1["choices"][0]["message"]
    assert r1["choices"][0]["finish_reason"] == "tool_calls" and m1["content"] is None and m1["reasoning_content"] == "need data"
    assert m1["tool_calls"][0]["function"] == {"name": "lookup", "arguments": '{"k": 1}'}
    # the client echoes the assistant message (without the reasoning) and adds the tool's result
    msgs += [{"role": "assistant", "content": None, "tool_calls": m1["tool_calls"]},
             {"role": "tool", "tool_call_id": m1["tool_calls"][0]["id"], "content": "k = 42"}]
    r2 = svc.chat({"messages": msgs, "tools": tools}, session_key="s")
    assert r2["choices"][0]["message"]["content"] == "It is 42." and r2["choices"][0]["finish_reason"] == "stop"
    smp = svc.finish_session("s", reward=1.0)
    full = TOK.decode(smp.tokens)
    assert len(svc.forest.sessions) == 1 and smp.weight_versions == [7]          # ONE session: the echo was recognised
    assert "<think>need data</think><tool_call>" in full and "k = 42" in full and full.rstrip().endswith("It is 42.")
    assert '"lookup"' in full.split("what is k?")[0]                              # the tool list is part of the prompt
    gen_text = TOK.decode([t for t, m_ in zip(smp.tokens[-smp.response_length:], smp.loss_mask) if m_])
    assert gen_text == '<think>need data</think><tool_call>{"name": "lookup", "arguments": {"k": 1}}</tool_call>It is 42.'
