"""A tool-using environment end to end: the policy may call a calculator tool, sees its result as a tool turn and
must end with ``Answer: <number>``; the reward is 1 for the right number.  Runs on a CPU with the tiny preset
(random weights, so rewards are noise: the point is the wiring).

    python examples/agentic_calculator.py
"""
import os
import re
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout

from relax_b200.models.config import get_config
from relax_b200.rollout import agentic as A
from relax_b200.rollout.engine import RolloutEngine, SamplingParams


@A.register_env("calculator")
class CalculatorEnv:
    def __init__(self, a: int = 17, b: int = 25):
        self.a, self.b = a, b

    def reset(self):
        return [{"role": "system", "content": "Use calc(<expr>) to compute; finish with 'Answer: <number>'."},
                {"role": "user", "content": f"What is {self.a} * {self.b}?"}]

    def step(self, text: str):
        m = re.search(r"Answer:\s*(-?\d+)", text)
        if m:
            return None, float(int(m.group(1)) == self.a * self.b), True
        c = re.search(r"calc\(([-+*/ 0-9()]+)\)", text)
        if c:
            try:
                return str(eval(c.group(1), {"__builtins__": {}})), 0.0, False   # digits and operators only
            except Exception:
                return "error", 0.0, False
        return "Call calc(...) or give the answer.", 0.0, False


def main():
    cfg = get_config("tiny")
    engine = RolloutEngine(cfg, device="cpu", num_kv_blocks=256, block_size=16, seed=0)
    tok = A.Tokenizer(encode=lambda s: [3 + (b % (cfg.vocab_size - 3)) for b in s.encode()],
                      decode=lambda ids: bytes((i - 3) % 256 for i in ids).decode("latin-1"))
    gen = A.engine_generate_fn(engine, SamplingParams(temperature=1.0, max_new_tokens=24))
    envs = [A.make_env("calculator", a=3 + i, b=7) for i in range(4)]
    sessions = A.run_episodes(envs, gen, tok, max_turns=3, max_new_tokens=24, max_context=512)
    for s in sessions:
        print(f"session {s.sid}: turns={s.turns} reward={s.reward} tokens={len(s.tokens)} trained={sum(s.loss_mask)}")
    return sessions


if __name__ == "__main__":
    main()
