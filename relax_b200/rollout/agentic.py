"""Agentic (multi-turn, tool-using) rollout.

An episode alternates model turns and environment turns (tool results, user replies).  The whole
conversation is ONE training sample: prompt and environment tokens carry loss mask 0, model tokens
carry mask 1 and their sampling log-probs, so the trainer sees exactly the tokens the engine
produced.  Every model turn re-submits "conversation so far" - the session keeps the token ids it
already has (no re-tokenisation of generated text, whose tokenisation need not round-trip) and the
engine's group prefix sharing turns the re-submission into a cache hit.

Pieces (relax/agentic/: ``rollout.py`` resident pipeline, ``session/state.py`` ``SessionForest``,
``session/service.py`` chat API, admission control):

* :class:`AgentEnv` - protocol of an environment: ``reset() -> messages``, ``step(text) -> (observation, reward, done)``.
* :class:`Session` / :class:`SessionForest` - token-level state of a conversation; ``fork`` branches an
  episode at a turn (tree search, best-of-n continuation) sharing the parent's prefix.
* :func:`run_episode` / :func:`run_episodes` - the loop; ``run_episodes`` advances many sessions in
  lock-step so that every engine call carries a full batch, bounded by an admission limit.
* env registry (:func:`register_env`) for ``--custom-env`` style lookup.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Protocol, Sequence, Tuple

from ..types import Sample, SampleStatus


class AgentEnv(Protocol):
    def reset(self) -> List[dict]: ...

    def step(self, assistant_text: str) -> Tuple[Optional[str], float, bool]: ...


_ENVS: Dict[str, Callable[..., AgentEnv]] = {}


def register_env(name: str):
    def deco(factory):
        _ENVS[name] = factory
        return factory

    return deco


def make_env(name: str, **kw) -> AgentEnv:
    if name not in _ENVS:
        raise KeyError(f"unknown environment {name!r}; registered: {sorted(_ENVS)}")
    return _ENVS[name](**kw)


@dataclass
class Tokenizer:
    encode: Callable[[str], List[int]]
    decode: Callable[[Sequence[int]], str]
    render_turn: Callable[[str, str], str] = lambda role, content: f"<|{role}|>\n{content}\n"
    generation_prompt: str = "<|assistant|>\n"


@dataclass
class Session:
    sid: int
    tokens: List[int] = field(default_factory=list)
    loss_mask: List[int] = field(default_factory=list)
    log_probs: List[float] = field(default_factory=list)
    weight_versions: List[int] = field(default_factory=list)
    prompt_len: int = 0
    turns: int = 0
    reward: float = 0.0
    done: bool = False
    truncated: bool = False
    parent: Optional[int] = None
    branch_point: int = 0          # tokens shared with the parent

    def append(self, toks: Sequence[int], mask: int, lps: Optional[Sequence[float]] = None):
        self.tokens += list(toks)
        self.loss_mask += [mask] * len(toks)
        self.log_probs += list(lps) if lps is not None else [0.0] * len(toks)

    def to_sample(self, group_index: Optional[int] = None, index: Optional[int] = None) -> Sample:
        rl = len(self.tokens) - self.prompt_len
        return Sample(group_index=group_index, index=index, tokens=list(self.tokens), response_length=rl,
                      loss_mask=self.loss_mask[self.prompt_len:], rollout_log_probs=self.log_probs[self.prompt_len:],
                      reward=self.reward, weight_versions=sorted(set(self.weight_versions)),
                      status=SampleStatus.TRUNCATED if self.truncated else SampleStatus.COMPLETED)


class SessionForest:
    """Sessions with parent links; a fork shares its parent's tokens up to the branch point."""

    def __init__(self):
        self.sessions: Dict[int, Session] = {}
        self._ids = itertools.count()

    def new(self) -> Session:
        s = Session(next(self._ids))
        self.sessions[s.sid] = s
        return s

    def fork(self, sid: int, at_tokens: Optional[int] = None) -> Session:
        p = self.sessions[sid]
        n = len(p.tokens) if at_tokens is None else at_tokens
        s = Session(next(self._ids), p.tokens[:n], p.loss_mask[:n], p.log_probs[:n], list(p.weight_versions),
                    p.prompt_len, p.turns, 0.0, False, False, parent=sid, branch_point=n)
        self.sessions[s.sid] = s
        return s

    def shared_prefix(self, a: int, b: int) -> int:
        ta, tb = self.sessions[a].tokens, self.sessions[b].tokens
        n = 0
        for x, y in zip(ta, tb):
            if x != y:
                break
            n += 1
        return n

    def children(self, sid: int) -> List[int]:
        return [s.sid for s in self.sessions.values() if s.parent == sid]


GenerateFn = Callable[[List[List[int]], int, List[int]], List[Tuple[List[int], List[float], str, List[int]]]]
"""``generate(prompts, max_new_tokens, group_keys) -> [(tokens, logprobs, finish_reason, weight_versions)]``"""


def engine_generate_fn(engine, sampling) -> GenerateFn:
    """Adapter over :class:`~relax_b200.rollout.engine.RolloutEngine`."""
    import dataclasses as _dc

    def gen(prompts, max_new, keys):
        sp = _dc.replace(sampling, max_new_tokens=max_new)
        res = engine.generate(prompts, sp, group_keys=keys)
        return [(list(r.output), list(r.logprobs), r.finish_reason, list(r.weight_versions)) for r in res]

    return gen


def run_episodes(envs: Sequence[AgentEnv], generate: GenerateFn, tok: Tokenizer, max_turns: int = 8,
                 max_new_tokens: int = 256, max_context: int = 4096, max_concurrent: Optional[int] = None,
                 forest: Optional[SessionForest] = None, admission=None) -> List[Session]:
    """Advance all episodes turn by turn; each engine call batches the sessions that still run (at most
    ``max_concurrent`` at a time).  With ``admission`` (a :class:`relax_b200.rollout.admission.AdmissionController`) an
    episode joins only once it holds a token lease for everything it may occupy in the KV cache - its prompt plus
    ``max_turns`` replies, capped by ``max_context`` - and gives the lease back when it ends; episodes are admitted in
    order, so a large one is not starved by small ones behind it."""
    forest = forest or SessionForest()
    sess: List[Session] = []
    for env in envs:
        s = forest.new()
        for m in env.reset():
            s.append(tok.encode(tok.render_turn(m["role"], m["content"])), 0)
        s.prompt_len = len(s.tokens)
        sess.append(s)
    live = list(range(len(envs)))
    leases: dict = {}
    pending = list(live) if admission is not None else []

    def admit():
        from .admission import reservation_tokens

        while pending:
            i = pending[0]
            need = min(max_context, reservation_tokens(sess[i].prompt_len, max_turns * max_new_tokens))
            # nothing admitted is running: wait for real (other users of the engines may free capacity; an aged waiter passes)
            lease = admission.acquire(need, timeout_s=None if not leases else 0.0)
            if lease is None:
                return
            leases[i] = lease
            pending.pop(0)

    while live:
        if admission is not None:
            admit()
            admitted = [i for i in live if i in leases]
        else:
            admitted = live
        wave = admitted[:max_concurrent] if max_concurrent else admitted
        prompts, budget = [], []
        for i in wave:
            s = sess[i]
            if s.turns == 0 or s.loss_mask[-1] == 0:
                gp = tok.encode(tok.generation_prompt)
                if len(s.tokens) + len(gp) < max_context:
                    s.append(gp, 0)
                else:
                    s.truncated = s.done = True
            room = 0 if s.done else max_context - len(s.tokens)
            budget.append(max(0, min(max_new_tokens, room)))
            prompts.append(list(s.tokens))
        runnable = [(i, p, b) for i, p, b in zip(wave, prompts, budget) if b > 0]
        for i, _, b in zip(wave, prompts, budget):
            if b <= 0:
                sess[i].truncated = sess[i].done = True
        if runnable:
            outs = generate([p for _, p, _ in runnable], max(b for _, _, b in runnable), [sess[i].sid for i, _, _ in runnable])
            for (i, _, b), (toks, lps, reason, versions) in zip(runnable, outs):
                s = sess[i]
                toks, lps = toks[:b], lps[:b]
                s.append(toks, 1, lps)
                s.weight_versions += versions
                s.turns += 1
                obs, reward, done = envs[i].step(tok.decode(toks))
                s.reward += reward
                if done or s.turns >= max_turns:
                    s.done = True
                    s.truncated = not done
                elif obs is not None:
                    ot = tok.encode(tok.render_turn("tool", obs))
                    if len(s.tokens) + len(ot) >= max_context:   # no room for the observation and a reply to it
                        s.truncated = s.done = True
                    else:
                        s.append(ot, 0)
        if admission is not None:
            for i in [i for i in live if sess[i].done and i in leases]:
                admission.release(leases.pop(i))
        live = [i for i in live if not sess[i].done]
    return sess


def run_episode(env: AgentEnv, generate: GenerateFn, tok: Tokenizer, **kw) -> Session:
    return run_episodes([env], generate, tok, **kw)[0]


# --------------------------------------------------------------------------- as a rollout generate function
_CODEC = None


def set_codec(codec) -> None:
    """Text codec (``data.tokenizer``) used by :func:`env_generate`; defaults to the byte-level codec."""
    global _CODEC
    _CODEC = codec


def env_generate(engine, samples, sampling_params):
    """Multi-turn, tool-using rollouts behind the single-turn interface of the training loop:
    ``--custom-generate-function-path relax_b200.rollout.agentic:env_generate``.

    Every sample names its environment in ``metadata["env"]`` (``{"name": ..., **kwargs}``; the registry of
    :func:`register_env`), optionally ``max_turns`` / ``max_new_tokens``.  The sample's prompt is replaced by the
    environment's opening messages; the returned sample carries the whole conversation, a loss mask that covers the
    model's own tokens only, the rollout log-probs of those tokens and the episode reward (so no reward function runs
    afterwards)."""
    from ..data.tokenizer import ByteCodec

    codec = _CODEC or ByteCodec(engine.cfg.vocab_size)
    tok = Tokenizer(encode=codec.encode, decode=codec.decode)
    envs, turns, new_tokens = [], 8, sampling_params.max_new_tokens
    for s in samples:
        spec = dict((s.metadata or {}).get("env") or {})
        if "name" not in spec:
            raise ValueError("env_generate: sample.metadata['env'] = {'name': ..., **kwargs} is required")
        turns = int((s.metadata or {}).get("max_turns", turns))
        envs.append(make_env(spec.pop("name"), **spec))
    max_ctx = getattr(engine, "max_model_len", None) or 4096
    admission = None
    if getattr(engine, "bm", None) is not None:          # an in-process engine: lease against its KV capacity
        admission = getattr(engine, "_admission", None)
        if admission is None:
            from .admission import AdmissionController

            admission = engine._admission = AdmissionController.for_engine(engine)
    sessions = run_episodes(envs, engine_generate_fn(engine, sampling_params), tok, max_turns=turns,
                            max_new_tokens=new_tokens, max_context=max_ctx, admission=admission)
    for s, sess in zip(samples, sessions):
        done = sess.to_sample(s.group_index, s.index)
        s.tokens, s.response_length, s.loss_mask = done.tokens, done.response_length, done.loss_mask
        s.rollout_log_probs, s.reward, s.status = done.rollout_log_probs, done.reward, done.status
        s.weight_versions = done.weight_versions
        s.response = codec.decode(done.tokens[len(done.tokens) - done.response_length:])
        s.metadata = dict(s.metadata or {}, turns=sess.turns)
    return samples


env_generate.manages_inference_permit = True
