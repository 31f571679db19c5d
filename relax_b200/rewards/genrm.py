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
