"""Generative reward model: a grader LLM reads the question, the reference answer and the policy's
answer, writes a verdict, and the verdict is parsed into a score (relax/components/genrm.py,
relax/distributed/ray/genrm.py, relax/utils/genrm_client.py, rule reward ``dapo_genrm``).  The grader
runs on its own engines; requests are spread round-robin, an engine that fails is skipped until
``recover`` brings it back, and unparsable verdicts score ``default``.
"""
from __future__ import annotations

import itertools
import re
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

DEFAULT_TEMPLATE = (
    "You are a strict grader.\nQuestion:\n{question}\n\nReference answer:\n{reference}\n\n"
    "Candidate answer:\n{answer}\n\nReply with 'Verdict: correct' or 'Verdict: incorrect', or 'Score: <0-10>'.\n")

_VERDICT = re.compile(r"verdict\s*[:\-]\s*(correct|incorrect|right|wrong|yes|no)", re.I)
_SCORE = re.compile(r"score\s*[:\-]\s*(-?\d+(?:\.\d+)?)(?:\s*/\s*(\d+(?:\.\d+)?))?", re.I)


def parse_verdict(text: str, default: float = 0.0) -> float:
    """Last verdict or score in the grader's text -> [0, 1]."""
    v = _VERDICT.findall(text)
    if v:
        return 1.0 if v[-1].lower() in ("correct", "right", "yes") else 0.0
    s = _SCORE.findall(text)
    if s:
        num, den = s[-1]
        den = float(den) if den else 10.0
        return min(1.0, max(0.0, float(num) / den)) if den > 0 else default
    return default


@dataclass
class JudgeEngine:
    generate_text: Callable[[List[str], int], List[str]]   # prompts, max_new_tokens -> completions
    healthy: bool = True


class GenRM:
    def __init__(self, engines: Sequence[JudgeEngine], template: str = DEFAULT_TEMPLATE, max_new_tokens: int = 256,
                 default: float = 0.0, parser: Callable[[str], float] = None):
        self.engines, self.template, self.max_new_tokens, self.default = list(engines), template, max_new_tokens, default
        self.parser = parser or (lambda t: parse_verdict(t, default))
        self._rr = itertools.count()
        self.failures = 0

    def _pick(self) -> Optional[JudgeEngine]:
        ok = [e for e in self.engines if e.healthy]
        return ok[next(self._rr) % len(ok)] if ok else None

    def recover(self, probe: Callable[[JudgeEngine], bool]):
        for e in self.engines:
            if not e.healthy and probe(e):
                e.healthy = True

    def score(self, questions: Sequence[str], references: Sequence[str], answers: Sequence[str]) -> List[float]:
        prompts = [self.template.format(question=q, reference=r, answer=a) for q, r, a in zip(questions, references, answers)]
        for _ in range(max(1, len(self.engines))):
            e = self._pick()
            if e is None:
                break
            try:
                outs = e.generate_text(prompts, self.max_new_tokens)
                return [self.parser(o) for o in outs]
            except Exception:  # noqa: BLE001
                e.healthy = False
                self.failures += 1
        return [self.default] * len(prompts)

    def reward_fn(self, detok: Callable[[Sequence[int]], str]) -> Callable:
        """A per-sample reward function for the rule-reward registry: judges ``sample.response`` (or the
        detokenised response tokens) against ``sample.label``."""
        def fn(sample) -> float:
            ans = sample.response or detok(sample.tokens[-sample.response_length:] if sample.response_length else [])
            return self.score([str(sample.prompt)], [str(sample.label)], [ans])[0]

        return fn


def engine_judge(engine, codec, temperature: float = 0.0, max_prompt_tokens: int = 2048) -> JudgeEngine:
    """A grader served by an in-house :class:`~relax_b200.rollout.engine.RolloutEngine` (the reference runs its
    grader on dedicated SGLang engines, relax/distributed/ray/genrm.py): prompts are tokenised with ``codec``,
    generated greedily (by default) and the completions detokenised for the verdict parser."""
    from ..rollout.engine import SamplingParams

    def generate_text(prompts: List[str], max_new_tokens: int) -> List[str]:
        ids = [codec.encode(p)[-max_prompt_tokens:] for p in prompts]
        sp = SamplingParams(temperature=temperature, max_new_tokens=max_new_tokens)
        res = engine.generate(ids, sp)
        return [codec.decode(r.output) for r in res]

    return JudgeEngine(generate_text)


def build_genrm(model_path: str, device, num_engines: int = 1, max_new_tokens: int = 64, codec=None, seed: int = 0) -> GenRM:
    """``--genrm-model-path``: a Hugging Face checkpoint directory (its config picks the architecture) or
    ``preset:<name>`` for a randomly initialised model of a built-in shape (tests).  One engine per ``num_engines``;
    they share the device with the caller (the grader runs between rollout and training)."""
    import torch

    from ..checkpoint import hf as H
    from ..data.tokenizer import build_codec
    from ..models.config import get_config
    from ..rollout.engine import RolloutEngine

    if model_path.startswith("preset:"):
        cfg, src = get_config(model_path.split(":", 1)[1]), None
    else:
        cfg, src = H.config_from_hf(model_path), model_path
    codec = codec or build_codec(src, cfg.vocab_size)
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[cfg.dtype]
    engines = []
    for i in range(max(1, num_engines)):
        eng = RolloutEngine(cfg, device=device, dtype=dt, num_kv_blocks=512, block_size=16, seed=seed + i,
                            eos_token_id=getattr(codec, "eos_token_id", None), use_cuda_graph=False, memory_saver=False)
        if src is not None:
            H.load_hf_into_rollout(src, cfg, eng.weights)
        else:
            g = torch.Generator(device="cpu").manual_seed(seed)
            eng.weights.flat.copy_((torch.randn(eng.weights.numel, generator=g) * 0.02).to(dt))
        engines.append(engine_judge(eng, codec))
    return GenRM(engines, max_new_tokens=max_new_tokens)


def build_remote_genrm(addrs: Sequence[str], codec, max_new_tokens: int = 64, timeout_s: float = 600.0) -> GenRM:
    """``--genrm-engine-addrs``: graders on engine servers of their own (``serve engine --hf-checkpoint <grader>`` on the
    GPUs set aside for them; the reference places its grader engines on ``--genrm-num-gpus`` dedicated GPUs,
    relax/distributed/ray/genrm.py).  Requests rotate over the servers; one that fails is skipped until it answers
    a probe again (:meth:`GenRM.recover`)."""
    from ..rollout.http_server import HTTPEngine

    if not addrs:
        raise ValueError("no grader address given")
    engines = [engine_judge(HTTPEngine(a if "://" in a else f"http://{a}", timeout_s), codec) for a in addrs]
    return GenRM(engines, max_new_tokens=max_new_tokens)
