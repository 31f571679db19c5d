"""Two-tier recovery driven by the controller (--use-fault-tolerance), with failures made on the host: a rollout that
raises once (global restart from the latest checkpoint, the run completes), a role that never recovers (the run stops
after --max-global-restart), and a two-rank job in which one rank reports a failure between steps (both restart together before the next step)."""
import json
import os

import pytest
import torch

from relax_b200.checkpoint import dist_ckpt
from tests._mp import run_distributed

COMMON = ["--model-name", "tiny", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
          "--rollout-max-prompt-len", "8", "--rollout-max-response-len", "8", "--lr", "1e-4", "--max-tokens-per-gpu", "256",
          "--colocate", "--use-fault-tolerance"]


def _controller(argv):
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    return Controller(parse_args(argv), device="cpu")


def test_rollout_failure_restarts_globally_from_the_checkpoint(tmp_path):
    save = str(tmp_path / "ckpt")
    ctl = _controller(COMMON + ["--num-rollout", "4", "--save", save, "--save-interval", "1", "--max-global-restart", "2"])
    gen, calls = ctl.runner.generate, {"n": 0}

    def flaky(rid):
        calls["n"] += 1
        if calls["n"] == 3:                      # the third rollout (rollout id 2) dies once
            raise RuntimeError("injected engine failure")
        return gen(rid)

    ctl.runner.generate = flaky
    hist = ctl.training_loop()
    assert ctl.restarts == {"inplace": 0, "global": 1}
    assert ctl.health_mgr.events[0][:2] == ("rollout", "global")
    assert len(hist) == 4 and ctl.runner.rollout_id == 4          # rollout 2 was redone after the restart
    assert dist_ckpt.read_latest_iteration(save) == 3
    assert ctl.runner.engine.bm.num_free >= ctl.runner.engine.bm.num_blocks - 1     # the aborted requests' blocks came back
    st = ctl.health.status()
    assert st["actor"]["healthy"] and st["rollout"]["healthy"] and st["rollout"]["restarts"] == 1


def test_a_role_that_keeps_failing_stops_the_run(tmp_path):
    ctl = _controller(COMMON + ["--num-rollout", "3", "--max-global-restart", "2"])

    def dead(rid):
        raise RuntimeError("engine is gone")

    ctl.runner.generate = dead
    with pytest.raises(RuntimeError, match="giving up after 2 global restarts"):
        ctl.training_loop()
    assert ctl.restarts["global"] == 2


def _two_rank_worker(rank, world):
    ctl = _controller(COMMON + ["--num-rollout", "3", "--rollout-batch-size", "4", "--global-batch-size", "8"])
    step, calls = ctl.runner.step, {"n": 0}

    def step_then_report():
        m = step()
        calls["n"] += 1
        if rank == 1 and calls["n"] == 1:        # between steps, on rank 1 only: its engine monitor reports a dead engine
            ctl.health.report_error("rollout", "engine 0 failed its health checks")
        return m

    ctl.runner.step = step_then_report
    hist = ctl.training_loop()
    return len(hist), ctl.restarts["global"], ctl.runner.rollout_id


def test_a_failure_reported_on_one_rank_between_steps_restarts_every_rank():
    out = run_distributed(_two_rank_worker, 2, timeout=300)
    assert out[0] == out[1] == (3, 1, 3)
