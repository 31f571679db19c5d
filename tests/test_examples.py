"""The recipes under examples/ stay in step with the flag table, and the Python example runs (CPU)."""
import os
import re
import shlex
import subprocess
import sys

import pytest

from relax_b200.config.arguments import parse_args

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EX = os.path.join(ROOT, "examples")


def _train_flags(path):
    text = open(path).read().replace("\\\n", " ")
    out = []
    for line in text.splitlines():
        if "relax_b200.entrypoints.train" in line:
            toks = shlex.split(line.split("relax_b200.entrypoints.train", 1)[1])
            out.append([t for t in toks if t != "$@"])
    return out


@pytest.mark.parametrize("name", sorted(f for f in os.listdir(EX) if f.endswith(".sh")))
def test_recipe_flags_parse(name):
    cmds = _train_flags(os.path.join(EX, name))
    assert cmds, name
    for flags in cmds:
        a = parse_args(flags)
        assert a.model_name


def test_readme_lists_every_recipe():
    readme = open(os.path.join(EX, "README.md")).read()
    for f in os.listdir(EX):
        if f != "README.md":
            assert f"`{f}`" in readme, f


def test_agentic_example_runs():
    r = subprocess.run([sys.executable, os.path.join(EX, "agentic_calculator.py")], capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stderr[-2000:]
    assert len(re.findall(r"session \d+: turns=", r.stdout)) == 4
