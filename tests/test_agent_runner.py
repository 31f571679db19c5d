"""External agent programs: the launcher daemon's ownership protocol, the active-time budget, the output contract,
and a rollout batch produced by real agent processes talking to the chat endpoint of a CPU engine."""
import json
import os
import sys
import textwrap
import time

import pytest

from relax_b200.rollout import agent_runner as R


@pytest.fixture(scope="module")
def daemon(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("launcher") / "l.sock")
    R.ensure_launcher_daemon(path)
    yield path
    R.stop_launcher_daemon(path)


def _agent(daemon, tmp_path, command, timeout_s=30.0, payload=None, **kw):
    spec = R.AgentSpec(command, str(tmp_path), {"EXTRA": "yes"}, timeout_s)
    return R.ManagedAgent(daemon, spec, "sess-1", "g7", payload or {"prompt": "hi"}, "http://127.0.0.1:1", **kw)


def test_session_output_forms():
    o = R.SessionOutput.from_text('{"reward": 1.5, "metadata": {"k": 1}}')
    assert o.reward == 1.5 and o.metadata == {"k": 1} and o.scalar_reward() == 1.5
    assert R.SessionOutput.from_text('{"reward": {"score": 0.25, "parts": [1]}}').scalar_reward() == 0.25
    assert R.SessionOutput.from_text("  ").reward is None
    recs = R.SessionOutput.from_text('{"name": "a", "messages": [{"role": "user", "content": "x"}], "reward": 1}\n'
                                     '{"name": "b", "messages": [{"role": "assistant", "content": "y"}]}')
    assert [r["name"] for r in recs.records] == ["a", "b"] and recs.records[0]["reward"] == 1
    for bad in ('[1, 2]', '{"reward": "high"}', '{"name": "a", "messages": []}\n{"name": "a", "messages": []}',
                '{"messages": [{"role": "user"}]}'):
        with pytest.raises(TypeError):
            R.SessionOutput.from_text(bad)
    with pytest.raises(ValueError):
        R.AgentSpec("  ", "/tmp")
    with pytest.raises(ValueError):
        R.AgentSpec("true", "/definitely/not/here")


def test_agent_sees_its_environment_and_reports_a_reward(daemon, tmp_path):
    cmd = (f"{sys.executable} -c \"import json, os; p = json.load(open(os.environ['RELAX_INPUT_JSON'])); "
           "json.dump({'reward': len(p['prompt']), 'metadata': {'sid': os.environ['RELAX_SESSION_ID'], 'grp': os.environ['RELAX_GROUP_ID'], "
           "'url': os.environ['RELAX_BASE_URL'], 'extra': os.environ['EXTRA'], 'mode': os.environ['RELAX_ROLLOUT_MODE'], "
           "'cwd': os.getcwd()}}, open(os.environ['RELAX_OUTPUT_JSON'], 'w'))\"")
    a = _agent(daemon, tmp_path, cmd, payload={"prompt": "four"}).start()
    out = a.wait()
    md = out.metadata
    assert out.reward == 4 and md["sid"] == "sess-1" and md["grp"] == "g7" and md["extra"] == "yes" and md["mode"] == "train"
    assert md["url"] == "http://127.0.0.1:1" and os.path.realpath(md["cwd"]) == os.path.realpath(str(tmp_path))
    assert "exit_at" in md["agent_events"] and not os.path.exists(a.dir)          # the scratch directory is gone


def test_failures_are_agent_errors_with_the_log_tail(daemon, tmp_path):
    a = _agent(daemon, tmp_path, "echo about to fail; exit 3").start()
    with pytest.raises(R.AgentExecutionError, match=r"status 3[\s\S]*about to fail"):
        a.wait()
    a = _agent(daemon, tmp_path, "echo '{not json' > $RELAX_OUTPUT_JSON").start()
    with pytest.raises(R.AgentExecutionError, match="invalid output"):
        a.wait()


def test_timeout_kills_the_whole_process_group_and_pauses_while_gated(daemon, tmp_path):
    mark = tmp_path / "child.pid"
    # the agent starts a background child and sleeps; both must be gone after the timeout
    a = _agent(daemon, tmp_path, f"sleep 60 & echo $! > {mark}; sleep 60", timeout_s=0.6).start(active=False)
    time.sleep(1.0)                      # gated: the clock does not run, the agent is still alive
    assert a.remaining_s == pytest.approx(0.6) and not a._exited.is_set()
    a.set_active(True)
    t0 = time.monotonic()
    with pytest.raises(R.AgentExecutionError, match="timed out"):
        a.wait()
    assert time.monotonic() - t0 < 5.0
    child = int(mark.read_text())
    deadline = time.monotonic() + 3.0
    while time.monotonic() < deadline:
        try:
            os.kill(child, 0)
        except ProcessLookupError:
            break
        time.sleep(0.05)
    else:
        pytest.fail("the agent's background child survived")


def test_owner_terminate_is_not_an_error(daemon, tmp_path):
    a = _agent(daemon, tmp_path, "sleep 60").start()
    t0 = time.monotonic()
    a.terminate()
    assert a._exited.is_set() and time.monotonic() - t0 < 5.0


AGENT = textwrap.dedent('''
    import json, os, urllib.request
    inp = json.load(open(os.environ["RELAX_INPUT_JSON"]))
    if inp["metadata"].get("crash"):
        raise SystemExit(2)
    msgs = [{"role": "user", "content": inp["prompt"]}]
    for turn in range(2):
        req = urllib.request.Request(os.environ["RELAX_BASE_URL"] + "/v1/chat/completions",
                                     data=json.dumps({"messages": msgs, "max_tokens": 5}).encode(),
                                     headers={"Content-Type": "application/json", "X-Session-Id": os.environ["RELAX_SESSION_ID"]})
        reply = json.loads(urllib.request.urlopen(req, timeout=120).read())["choices"][0]["message"]["content"]
        msgs += [{"role": "assistant", "content": reply}, {"role": "user", "content": "tool says: %d" % turn}]
    json.dump({"reward": float(inp["index"]), "metadata": {"tool_calls": 2}}, open(os.environ["RELAX_OUTPUT_JSON"], "w"))
''')


def test_rollout_batch_from_agent_processes(tmp_path):
    import torch

    from relax_b200.data.tokenizer import ByteCodec
    from relax_b200.models.config import get_config
    from relax_b200.rollout.agent_pipeline import AgentPipeline
    from relax_b200.rollout.agentic import Tokenizer
    from relax_b200.rollout.engine import RolloutEngine, SamplingParams
    from relax_b200.types import Sample, SampleStatus

    (tmp_path / "agent.py").write_text(AGENT)
    cfg = get_config("tiny")
    eng = RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=256, block_size=8, max_model_len=512)
    codec = ByteCodec(cfg.vocab_size)
    tok = Tokenizer(encode=codec.encode, decode=codec.decode)
    sock = str(tmp_path / "l.sock")
    pipe = AgentPipeline(R.AgentSpec(f"{sys.executable} agent.py", str(tmp_path), {}, 120.0), tok, concurrency=4,
                         admission=True, socket_path=sock)
    samples = []
    for g in range(3):
        for i in range(2):
            samples.append(Sample(group_index=g, index=g * 2 + i, prompt=f"question {g}", tokens=codec.encode(f"question {g}"),
                                  metadata={"crash": g == 1 and i == 1}))
    try:
        out = pipe.run(eng, samples, SamplingParams(temperature=1.0, max_new_tokens=5))
    finally:
        R.stop_launcher_daemon(sock)
    ok = [s for s in out if s.group_index != 1]
    for s in ok:
        assert s.status in (SampleStatus.COMPLETED, SampleStatus.TRUNCATED) and s.reward == float(s.index)
        assert s.metadata["turns"] == 2 and s.metadata["tool_calls"] == 2
        assert len(s.loss_mask) == s.response_length == len(s.rollout_log_probs)
        assert 0 < sum(s.loss_mask) <= 10 and s.loss_mask[-1] == 1                     # two model turns of <= 5 tokens
        gen = [lp for lp, m in zip(s.rollout_log_probs, s.loss_mask) if m]
        assert all(lp <= 0 for lp in gen) and any(lp < 0 for lp in gen)
        assert "tool says: 0" in codec.decode(s.tokens) and s.weight_versions == [eng.weight_version]
    # the crashed agent takes its whole prompt group out of the loss
    for s in [s for s in out if s.group_index == 1]:
        assert s.remove_sample and s.status == SampleStatus.FAILED and s.loss_mask == [0] and s.reward == 0.0
    assert "status 2" in out[3].metadata["agent_error"]
    assert pipe.stats["agentic/failed_groups"] == 1.0 and pipe.stats["agentic/sessions"] == 6.0
    assert pipe.stats["agentic/admission_peak_reserved"] > 0
    # the engine is usable by its owner again after the call
    assert len(eng.generate([codec.encode("again")], SamplingParams(max_new_tokens=3))[0].output) == 3


def test_use_agentic_rollout_through_the_controller(tmp_path):
    """``--use-agentic-rollout --agent-command ...``: a colocated GRPO step trained on what agent processes produced."""
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller
    from relax_b200.rollout import agent_pipeline

    (tmp_path / "agent.py").write_text(AGENT)
    f = tmp_path / "prompts.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": f"task {i}", "label": None}) for i in range(2)) + "\n")
    with pytest.raises(ValueError, match="--agent-command"):
        parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--use-agentic-rollout"])
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "5", "--rollout-max-prompt-len", "256", "--prompt-data", str(f),
                    "--input-key", "prompt", "--use-agentic-rollout", "--agent-command", f"{sys.executable} agent.py",
                    "--agent-cwd", str(tmp_path), "--agent-timeout", "120", "--agent-env", "A=1", "B=two words",
                    "--agentic-program-admission", "--disable-rewards-normalization"])
    assert a.custom_generate_function_path.endswith("agent_pipeline:command_generate") and a.agentic_concurrency == 2
    c = Controller(a, device="cpu")
    try:
        assert agent_pipeline._PIPELINE.spec.env == {"A": "1", "B": "two words"} and agent_pipeline._PIPELINE.use_admission
        m = c.runner.step()
        assert m["agentic/sessions"] == 4.0 and m["agentic/failed_groups"] == 0.0 and m["agentic/turns_mean"] == 2.0
        assert "loss" in m and m["agentic/admission_peak_reserved"] > 0
    finally:
        R.stop_launcher_daemon(agent_pipeline._PIPELINE.socket_path)


def test_custom_group_advantage_for_agent_rollouts(tmp_path):
    """``--agentic-custom-advantage-path``: user code turns a prompt group's samples into advantages; the trainer uses
    them as they are (the estimator's group normalisation is bypassed)."""
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller
    from relax_b200.rollout import agent_pipeline

    (tmp_path / "agent.py").write_text(AGENT)
    (tmp_path / "adv.py").write_text("def rank_in_group(samples):\n    return [float(i) - 0.5 for i, _ in enumerate(samples)]\n")
    f = tmp_path / "prompts.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": f"task {i}", "label": None}) for i in range(2)) + "\n")
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "5", "--rollout-max-prompt-len", "256", "--prompt-data", str(f),
                    "--input-key", "prompt", "--use-agentic-rollout", "--agent-command", f"{sys.executable} agent.py",
                    "--agent-cwd", str(tmp_path), "--agentic-custom-advantage-path", f"{tmp_path / 'adv.py'}:rank_in_group"])
    c = Controller(a, device="cpu")
    try:
        samples = c.runner.generate(0)
        assert [s.custom_advantage for s in samples] == [-0.5, 0.5, -0.5, 0.5]
        m = c.runner.step()
        assert abs(m["rollout/advantages"]) < 1e-6 and "loss" in m          # mean of -0.5 / +0.5 over equally long responses
    finally:
        R.stop_launcher_daemon(agent_pipeline._PIPELINE.socket_path)


def test_no_agent_outlives_the_daemon(tmp_path):
    """When the daemon leaves (its owner stopped it or died), the agents it started are ended with it."""
    sock = str(tmp_path / "d.sock")
    R.ensure_launcher_daemon(sock)
    mark = tmp_path / "pid"
    a = R.ManagedAgent(sock, R.AgentSpec(f"echo $$ > {mark}; sleep 60", str(tmp_path), {}, 120.0), "s", "g", {}, "http://127.0.0.1:1").start()
    deadline = time.monotonic() + 5
    while not mark.exists() and time.monotonic() < deadline:
        time.sleep(0.02)
    pid = int(mark.read_text())
    os.kill(pid, 0)                                   # alive
    R.stop_launcher_daemon(sock)
    deadline = time.monotonic() + 6
    while time.monotonic() < deadline:
        try:
            os.kill(pid, 0)
        except ProcessLookupError:
            break
        time.sleep(0.05)
    else:
        pytest.fail("the agent survived its daemon")
    with pytest.raises(R.AgentExecutionError):
        a.wait(poll_s=5)


def test_evaluation_runs_through_the_agent_pipeline(tmp_path):
    """Held-out prompts are evaluated the way the policy is trained: agent processes (in eval mode) produce the samples."""
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller
    from relax_b200.rollout import agent_pipeline

    (tmp_path / "agent.py").write_text(AGENT.replace('"tool_calls": 2}', '"tool_calls": 2, "mode": os.environ["RELAX_ROLLOUT_MODE"]}'))
    f = tmp_path / "prompts.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": f"task {i}", "label": None}) for i in range(2)) + "\n")
    ev = tmp_path / "eval.jsonl"
    ev.write_text("\n".join(json.dumps({"prompt": f"held out {i}", "label": None}) for i in range(3)) + "\n")
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "5", "--rollout-max-prompt-len", "256", "--prompt-data", str(f),
                    "--input-key", "prompt", "--use-agentic-rollout", "--agent-command", f"{sys.executable} agent.py",
                    "--agent-cwd", str(tmp_path), "--eval-prompt-data", "heldout", str(ev), "--eval-interval", "1"])
    c = Controller(a, device="cpu")
    try:
        seen = []
        real = agent_pipeline._PIPELINE._export

        def spy(s, sess, out):
            seen.append(out.metadata.get("mode"))
            return real(s, sess, out)

        agent_pipeline._PIPELINE._export = spy
        m = c.runner.step()
        assert "eval" in seen and "train" in seen
        ek = [k for k in m if k.startswith("eval/heldout")]
        assert ek and any("reward" in k or "score" in k or "mean" in k for k in ek), sorted(m)
    finally:
        R.stop_launcher_daemon(agent_pipeline._PIPELINE.socket_path)
