"""Rollouts produced by external agent programs (``--use-agentic-rollout``).

Each sample of a rollout batch becomes one *session*: an agent process (:mod:`relax_b200.rollout.agent_runner`) is
started for it, talks to the policy through the chat endpoint (:mod:`relax_b200.rollout.openai_api`) under its session
id, and exits with a reward.  What the endpoint recorded for that session - the token ids the engine saw and produced,
a loss mask over the model's own tokens, their sampling log-probs, the weight versions - is the training sample.  The
reference's counterpart is its resident agentic pipeline (relax/agentic/rollout.py ``AgenticResidentPipeline`` :120,
``_run_group`` :74; relax/agentic/pipeline/runtime.py for the backend attempts; relax/agentic/pipeline/reward.py for
the reward hand-over).

How the pieces sit together here:

* the engine is owned by ONE loop thread for the length of the call (:class:`~relax_b200.rollout.http_server.EngineServer`
  without its HTTP front end); completions of different sessions arrive on HTTP handler threads and join the running
  batch at the next scheduler iteration, so forty agents that think at different speeds still decode together;
* every completion first takes a token lease from the :class:`~relax_b200.rollout.admission.AdmissionController`
  (context + what it may generate, against the KV capacity); while it waits the agent's time budget is paused;
* at most ``concurrency`` sessions are resident; a prompt group whose agent fails (non-zero status, timeout, bad
  output, no completion recorded) is dropped as a whole: its samples come back with ``remove_sample`` set, which
  zeroes their loss mask, so a crashed tool never turns into a gradient.

``command_generate`` has the signature of a custom generate function; the controller installs it when
``--use-agentic-rollout`` is given (``configure`` receives the parsed flags).
"""
from __future__ import annotations

import itertools
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional

from ..types import SampleStatus
from .agent_runner import AgentExecutionError, AgentLauncher, AgentSpec, ManagedAgent, SessionOutput
from .agentic import Tokenizer


def rollout_mode_is_train(mode: str) -> bool:
    return mode == "train"


class AgentPipeline:
    def __init__(self, spec: AgentSpec, tok: Tokenizer, concurrency: int = 32, admission: bool = True,
                 admission_headroom: float = 0.9, admission_pressure: float = 0.92, admission_max_wait_s: float = 30.0,
                 max_context: Optional[int] = None, socket_path: Optional[str] = None, rollout_mode: str = "train",
                 tool_call_parser: Optional[str] = None, reasoning_parser: Optional[str] = None,
                 custom_advantage_path: Optional[str] = None):
        self.spec, self.tok, self.concurrency = spec, tok, max(1, int(concurrency))
        self.use_admission, self.headroom = admission, admission_headroom
        self.pressure, self.max_wait_s = admission_pressure, admission_max_wait_s
        self.max_context, self.socket_path, self.rollout_mode = max_context, socket_path, rollout_mode
        self.tool_call_parser, self.reasoning_parser = tool_call_parser, reasoning_parser
        # --agentic-custom-advantage-path: ``fn(samples of one prompt group) -> one number per sample``; the numbers become
        # the samples' advantages instead of the estimator's (relax/agentic/pipeline/reward.py custom_advantage_func)
        self.custom_advantage = None
        if custom_advantage_path:
            from .custom_generate import load_function

            self.custom_advantage = load_function(custom_advantage_path, 1, "custom advantage function")
        self.stats: Dict[str, float] = {}
        self._seq = itertools.count(1)

    # ------------------------------------------------------------------ one rollout batch
    def run(self, engine, samples: list, sampling, rollout_mode: Optional[str] = None) -> list:
        from .admission import AdmissionController
        from .http_server import EngineServer
        from .openai_api import ChatService, serve

        mode = rollout_mode or self.rollout_mode            # "eval": agents see RELAX_ROLLOUT_MODE=eval, no custom advantages
        agents: Dict[str, ManagedAgent] = {}
        adm = None
        if self.use_admission and getattr(engine, "bm", None) is not None:
            adm = AdmissionController.for_engine(engine, headroom=self.headroom, pressure_guard=self.pressure,
                                                 max_wait_s=self.max_wait_s)

        def on_gate(key, waiting):
            a = agents.get(key)
            if a is not None:
                a.set_active(not waiting)

        backend = EngineServer(engine, http=False)
        chat = ChatService(backend.generate_fn(sampling), self.tok, max_context=self.max_context or getattr(engine, "max_model_len", None) or 8192,
                           concurrent=True, admission=adm, on_gate=on_gate, tool_call_parser=self.tool_call_parser,
                           reasoning_parser=self.reasoning_parser)
        httpd, url = serve(chat)
        launcher = AgentLauncher(self.spec, url, self.socket_path)
        t0 = time.perf_counter()
        results: Dict[int, tuple] = {}
        try:
            def one(i_s):
                i, s = i_s
                sid = f"s{next(self._seq)}-{s.group_index}-{s.index if s.index is not None else i}"
                payload = {"prompt": s.prompt, "label": s.label, "metadata": s.metadata or {}, "group_index": s.group_index,
                           "index": s.index, "max_new_tokens": sampling.max_new_tokens}
                try:
                    a = ManagedAgent(launcher.socket_path, launcher.spec, sid, str(s.group_index), payload, url, mode)
                    agents[sid] = a
                    a.start()
                    out = a.wait()
                    results[i] = (sid, out, None)
                except (AgentExecutionError, OSError, TimeoutError) as e:
                    results[i] = (sid, None, e)
                finally:
                    agents.pop(sid, None)

            with ThreadPoolExecutor(max_workers=self.concurrency, thread_name_prefix="agent") as pool:
                list(pool.map(one, enumerate(samples)))
        finally:
            for a in list(agents.values()):
                a.terminate()
            httpd.shutdown()
            httpd.server_close()
            backend.close()
        failed_groups = set()
        for i, s in enumerate(samples):
            sid, out, err = results.get(i, (None, None, AgentExecutionError("the agent was never started")))
            sess = chat.by_key.pop(sid, None) if sid else None
            if err is None and (sess is None or not any(sess.loss_mask)) and not (out and out.records):
                err = AgentExecutionError("the agent exited without a single completion")
            if err is not None:
                failed_groups.add(s.group_index)
                s.metadata = dict(s.metadata or {}, agent_error=str(err)[:2000])
                continue
            self._export(s, sess, out)
        for s in samples:
            if s.group_index in failed_groups:
                self._drop(s)
        if self.custom_advantage is not None and rollout_mode_is_train(mode):
            groups: Dict[object, list] = {}
            for s in samples:
                if s.group_index not in failed_groups:
                    groups.setdefault(s.group_index, []).append(s)
            for g in groups.values():
                vals = list(self.custom_advantage(g))
                if len(vals) != len(g) or any(isinstance(v_, bool) or not isinstance(v_, (int, float)) for v_ in vals):
                    raise TypeError("the custom advantage function returns one number per sample of the group")
                for s, v_ in zip(g, vals):
                    s.custom_advantage = float(v_)
            for s in samples:
                if s.group_index in failed_groups:
                    s.custom_advantage = 0.0
        self.stats = {"agentic/sessions": float(len(samples)), "agentic/failed_groups": float(len(failed_groups)),
                      "agentic/wall_s": time.perf_counter() - t0,
                      "agentic/turns_mean": sum((s.metadata or {}).get("turns", 0) for s in samples) / max(1, len(samples))}
        if adm is not None:
            m = adm.metrics()
            self.stats.update({"agentic/admission_wait_mean_s": m["wait_mean_s"], "agentic/admission_bypassed": float(m["bypassed"]),
                               "agentic/admission_peak_reserved": float(m["peak_reserved"])})
        return samples

    # ------------------------------------------------------------------ sample export
    def _export(self, s, sess, out: SessionOutput):
        if out.records:
            toks, mask = self._tokens_of_messages(out.records[0]["messages"])
            plen = next((i for i, m in enumerate(mask) if m), len(toks))
            s.tokens, s.response_length = toks, len(toks) - plen
            s.loss_mask, s.rollout_log_probs = mask[plen:], None         # the text was not sampled here token by token
            rec = out.records[0]
            reward, md = rec.get("reward"), rec.get("metadata", {})
            turns = sum(1 for m in rec["messages"] if m.get("role") == "assistant")
        else:
            d = sess.to_sample(s.group_index, s.index)
            s.tokens, s.response_length, s.loss_mask = d.tokens, d.response_length, d.loss_mask
            s.rollout_log_probs, s.weight_versions = d.rollout_log_probs, d.weight_versions
            reward, md, turns = out.reward, out.metadata, sess.turns
        if isinstance(reward, dict):
            md = dict(md, reward_details=reward)
            reward = reward.get("reward", reward.get("score"))
        s.reward = None if reward is None else float(reward)          # None: the loop's reward function scores it
        s.status = SampleStatus.TRUNCATED if (sess is not None and sess.truncated) else SampleStatus.COMPLETED
        s.response = self.tok.decode(s.tokens[len(s.tokens) - s.response_length:])
        s.metadata = dict(s.metadata or {}, turns=turns, **{k: v for k, v in md.items() if k != "turns"})

    def _tokens_of_messages(self, messages: list):
        toks: List[int] = []
        mask: List[int] = []
        for m in messages:
            if m.get("role") == "assistant":
                head = self.tok.encode(self.tok.generation_prompt)
                body = self.tok.encode((m.get("content") or "") + "\n")
                toks += head + body
                mask += [0] * len(head) + [1] * len(body)
            else:
                t = self.tok.encode(self.tok.render_turn(m["role"], m.get("content") or ""))
                toks += t
                mask += [0] * len(t)
        return toks, mask

    @staticmethod
    def _drop(s):
        prompt = list(s.tokens) or [0]
        s.tokens, s.response_length = prompt + prompt[-1:], 1
        s.loss_mask, s.rollout_log_probs = [0], [0.0]
        s.reward, s.remove_sample, s.status = 0.0, True, SampleStatus.FAILED


# --------------------------------------------------------------------------- as a generate function
_PIPELINE: Optional[AgentPipeline] = None
_LOCK = threading.Lock()


def configure(args, codec=None) -> AgentPipeline:
    """Build the process-wide pipeline from the parsed flags (``--agent-command``, ``--agent-cwd``, ``--agent-env``,
    ``--agent-timeout``, ``--agentic-concurrency``, ``--agentic-program-admission`` and its knobs) and start the
    launcher daemon.  Called by the controller before the engines allocate their memory."""
    global _PIPELINE
    from ..data.tokenizer import ByteCodec
    from .agent_runner import ensure_launcher_daemon

    codec = codec or ByteCodec(getattr(args, "vocab_size", None) or 256)
    tok = Tokenizer(encode=codec.encode, decode=codec.decode)
    g = lambda k, d: getattr(args, k, d) if getattr(args, k, None) is not None else d
    with _LOCK:
        _PIPELINE = AgentPipeline(
            AgentSpec.from_args(args), tok, concurrency=g("agentic_concurrency", 32),
            admission=bool(g("agentic_program_admission", False)), admission_headroom=g("agentic_admission_headroom", 0.9),
            admission_pressure=g("agentic_admission_pressure_threshold", 0.92), admission_max_wait_s=g("agentic_admission_max_wait_s", 30.0),
            socket_path=ensure_launcher_daemon(), tool_call_parser=g("agentic_tool_call_parser", None),
            reasoning_parser=g("agentic_reasoning_parser", None), custom_advantage_path=g("agentic_custom_advantage_path", None))
    return _PIPELINE


def command_generate(engine, samples, sampling_params):
    """``fn(engine, samples, sampling_params) -> samples`` over the configured pipeline."""
    if _PIPELINE is None:
        raise RuntimeError("agent_pipeline.configure(args) has not run (--use-agentic-rollout with --agent-command / --agent-cwd)")
    return _PIPELINE.run(engine, samples, sampling_params)


def _command_generate_eval(engine, samples, sampling_params):
    if _PIPELINE is None:
        raise RuntimeError("agent_pipeline.configure(args) has not run")
    return _PIPELINE.run(engine, samples, sampling_params, rollout_mode="eval")


command_generate.eval_variant = _command_generate_eval
command_generate.manages_inference_permit = True
command_generate.stats = lambda: dict(_PIPELINE.stats) if _PIPELINE is not None else {}
