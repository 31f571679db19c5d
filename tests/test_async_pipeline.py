"""Fully-async / hybrid role loops with bounded staleness, gated weight updates, health and restart policy."""
import threading
import time

import pytest
import torch

from relax_b200.data.convert import convert_samples_to_train_data
from relax_b200.health.monitor import (HealthManager, HealthRegistry, RolloutHealthMonitor, maybe_inject_fault,
                                       restart_tier)
from relax_b200.orchestration.async_pipeline import AsyncPipeline, PipelineConfig, WeightChannel
from relax_b200.orchestration.registry import (ROLES_COLOCATE, ROLES_FULLY_ASYNC, Role, assign_ranks, process_role,
                                               satisfy_staleness)
from relax_b200.types import Sample


def test_staleness_gate_matches_rule():
    assert satisfy_staleness(None, 5, 0) and satisfy_staleness([], 5, 0)
    assert satisfy_staleness(["train_3"], 2, 0)            # 2 + 1 - 3 = 0
    assert not satisfy_staleness(["train_3"], 3, 0)        # would be 1 ahead
    assert satisfy_staleness(["train_3", "train_4"], 3, 1)
    assert not satisfy_staleness(["train_2", "train_4"], 4, 2)


def test_role_sets_by_mode():
    class C:
        debug_rollout_only = debug_train_only = False
        loss_type = "policy_loss"
        advantage_estimator = "grpo"
        fully_async = hybrid = true_on_policy_mode = False

    c = C()
    assert process_role(c) == (Role.actor, Role.rollout)           # colocate, no critic for grpo
    c.fully_async = True
    assert set(process_role(c)) == set(ROLES_FULLY_ASYNC) - {Role.critic}
    c.true_on_policy_mode = True
    assert Role.actor_fwd not in process_role(c)
    c.hybrid = True
    assert process_role(c) == (Role.actor, Role.rollout)
    c.hybrid, c.advantage_estimator, c.fully_async, c.true_on_policy_mode = False, "ppo", False, False
    assert process_role(c) == ROLES_COLOCATE
    c.debug_train_only = True
    assert process_role(c) == (Role.actor,)
    r = assign_ranks({"actor": (1, 4), "rollout": (1, 4)}, 8, colocate=False)
    assert r["actor"] == (0, 1, 2, 3) and r["rollout"] == (4, 5, 6, 7)
    r = assign_ranks({"actor": (1, 8), "rollout": (1, 8)}, 8, colocate=True)
    assert r["actor"] == r["rollout"] == tuple(range(8))


def _fake_parts(max_staleness, num_rollout=6, train_sleep=0.03, with_fwd=True):
    state = {"version": 0, "pushed": [], "recv": [], "trained": []}

    def generate(rid):
        out = []
        for g in range(2):
            for k in range(2):
                s = Sample(group_index=rid * 2 + g, index=(rid * 2 + g) * 2 + k, tokens=[1, 2, 3, 4 + k, 5], response_length=2,
                           reward=float(k), rollout_log_probs=[-1.0, -1.0], weight_versions=[state["version"]])
                out.append(s)
        return out

    def convert(samples):
        return convert_samples_to_train_data(samples, n_samples_per_prompt=2)

    def train(rid, batch):
        time.sleep(train_sleep)
        state["trained"].append((rid, batch))
        return {"loss": 0.0}

    def export():
        state["version"] += 1
        return {"v": state["version"]}

    fwd = (lambda b: [torch.full((r,), -0.5) for r in b["response_lengths"]]) if with_fwd else None
    ref = (lambda b: [torch.full((r,), -0.75) for r in b["response_lengths"]]) if with_fwd else None
    pipe = AsyncPipeline(PipelineConfig(num_rollout=num_rollout, max_staleness=max_staleness), generate_fn=generate,
                         convert_fn=convert, train_fn=train, export_weights_fn=export,
                         push_to_rollout_fn=lambda p: state["pushed"].append(p["v"]),
                         recv_weight_fn=lambda role, p: state["recv"].append((role.value, p["v"])), fwd_fn=fwd, ref_fn=ref)
    return pipe, state


@pytest.mark.parametrize("max_staleness", [0, 1, 2])
def test_fully_async_respects_staleness_and_feeds_every_role(max_staleness):
    pipe, st = _fake_parts(max_staleness)
    assert {l.role for l in pipe.loops} == {Role.rollout, Role.actor_fwd, Role.reference, Role.advantages, Role.actor}
    pipe.run(timeout=60)
    assert [rid for rid, _ in st["trained"]] == list(range(6))
    for rid, ver, unconsumed in pipe.rollout_started:
        # when rollout `rid` started the trainer had published at least rid - max_staleness - ... versions
        oldest = min([int(p.split("_")[1]) for p in unconsumed] + [rid])
        assert rid - oldest <= max_staleness
    for rid, batch in st["trained"]:
        assert batch["log_probs"][0] == [-0.5, -0.5] and batch["ref_log_probs"][0] == [-0.75, -0.75]
        assert len(batch["advantages"]) == 4 and len(batch["advantages"][0]) == 2
        # group-normalised rewards 0/1 -> -/+ 0.707..
        assert batch["advantages"][0][0] < 0 < batch["advantages"][1][0]
    assert st["pushed"] == [1, 2, 3, 4, 5, 6]
    assert ("actor_fwd", 1) in st["recv"] and all(r == "actor_fwd" for r, _ in st["recv"])   # the reference stays frozen
    assert pipe.queue.get_partition_list() == []


def test_hybrid_runs_forward_roles_inside_the_actor():
    cfg = PipelineConfig(num_rollout=3, max_staleness=1, hybrid=True)
    seen = []
    pipe = AsyncPipeline(cfg, generate_fn=lambda rid: [Sample(group_index=0, index=i, tokens=[1, 2, 3], response_length=1, reward=1.0 * i)
                                                       for i in range(2)],
                         convert_fn=lambda s: convert_samples_to_train_data(s, n_samples_per_prompt=2),
                         train_fn=lambda rid, b: seen.append(sorted(b)) or {}, export_weights_fn=lambda: {},
                         push_to_rollout_fn=lambda p: None, fwd_fn=lambda b: [], ref_fn=lambda b: [])
    assert {l.role for l in pipe.loops} == {Role.rollout, Role.actor}
    pipe.run(timeout=30)
    assert len(seen) == 3 and "log_probs" not in seen[0]


def test_role_failure_is_reported_not_hung():
    def bad_train(rid, batch):
        raise RuntimeError("boom")

    pipe, st = _fake_parts(1, num_rollout=2)
    pipe.train_fn = bad_train
    with pytest.raises((RuntimeError, TimeoutError)) as ei:
        pipe.run(timeout=5)
    assert "boom" in str(ei.value) or "still running" in str(ei.value)
    assert any(not v["healthy"] for v in pipe.health.status().values())
    pipe.stop()


def test_weight_channel_parks_rollout_during_update():
    ch = WeightChannel()
    order = []

    def rollout():
        for i in range(200):
            ch.park_if_requested()
            order.append("gen")
            time.sleep(0.001)

    t = threading.Thread(target=rollout)
    t.start()
    time.sleep(0.02)
    assert ch.request_update(timeout=5)
    n = len(order)
    time.sleep(0.05)
    assert len(order) == n                      # nothing generated while weights move
    ch.publish({"x": 1}, 1)
    ch.end_update()
    t.join(5)
    assert len(order) == 200 and ch.version == 1


def test_health_two_tier_restart_and_fatal():
    now = [0.0]
    reg = HealthRegistry(heartbeat_timeout=10.0, clock=lambda: now[0])
    log = []
    mgr = HealthManager(reg, restart_inplace=lambda n: log.append(("inplace", n)), restart_global=lambda n: log.append(("global", n)),
                        on_fatal=lambda m: log.append(("fatal", m)), max_global_restart=1)
    for n in ("actor", "rollout", "advantages"):
        reg.register(n)
    now[0] = 5.0
    reg.heartbeat("actor"); reg.heartbeat("rollout")
    now[0] = 12.0                                # advantages missed its heartbeat
    mgr.check_once()
    assert log == [("inplace", "advantages")]
    reg.report_error("rollout", "engine died")
    mgr.check_once()
    assert log[-1] == ("global", "rollout") and mgr.global_restarts == 1
    reg.report_error("actor", "nccl timeout")
    mgr.check_once()
    assert log[-1][0] == "fatal"
    assert restart_tier("advantages", 0) == "inplace" and restart_tier("advantages", 3) == "global"
    assert restart_tier("actor_fwd", 0) == "global"


def test_rollout_engine_monitor_and_fault_injection():
    class Eng:
        def __init__(self):
            self.ok = True

        def health(self):
            if not self.ok:
                raise ConnectionError("no answer")
            return True

    engines = {0: Eng(), 1: Eng()}
    recreated = []

    def recover(eid):
        engines[eid] = Eng()
        recreated.append(eid)

    mon = RolloutHealthMonitor(engines, recover, max_failures=2)
    mon.poll_once()
    assert recreated == []
    engines[1].ok = False
    mon.poll_once(); mon.poll_once()
    assert recreated == [1] and engines[1].ok
    assert not maybe_inject_fault(True, True, 1, mon)
    assert maybe_inject_fault(True, True, 2, mon)
    mon.poll_once(); mon.poll_once()
    assert recreated == [1, 0]


def test_partial_rollout_aborts_resumes_and_masks_offpolicy_tokens():
    """Over-sampling with early stop: groups still running when the batch is full are aborted into the rollout
    buffer with their partial responses, the next step continues them, and (with the mask flag) only the tokens of
    the current policy stay in the loss."""
    import torch

    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.orchestration.colocate import ColocateConfig, ColocatedGRPO
    from relax_b200.train.actor import TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig
    from relax_b200.types import SampleStatus

    torch.manual_seed(0)
    cfg = ColocateConfig(
        model=get_config("tiny"),
        train=TrainConfig(advantage_estimator="grpo", n_samples_per_prompt=2, global_batch_size=8, max_tokens_per_gpu=2048,
                          loss=LossConfig(eps_clip=0.2), optim=OptimizerConfig(lr=1e-5)),
        rollout_batch_size=4, over_sampling_batch_size=8, partial_rollout=True, mask_offpolicy_in_partial_rollout=True,
        prompt_len=8, max_response_len=160, temperature=1.0, rm_type="parity", eos_token_id=3, seed=0, rollout_seed=5,
        stop_token_ids=list(range(0, 1024, 48)), kv_blocks=512)     # responses end at random lengths: some groups are mid-way when 4 are done
    run = ColocatedGRPO(cfg)
    first = run.generate(0)
    assert len(first) == 8 and all(s.status in (SampleStatus.COMPLETED, SampleStatus.TRUNCATED) for s in first)
    st = run.sampling_stats
    assert st["aborted_samples"] > 0 and len(run.data_source.buffer) > 0
    partial = {s.index: s.response_length for g in run.data_source.buffer for s in g if s.status == SampleStatus.ABORTED}
    assert any(n > 0 for n in partial.values()), "at least one aborted sample had generated tokens"
    assert run.engine.bm.num_free == run.engine.bm.num_blocks
    second = run.generate(1)
    assert run.sampling_stats["resumed_samples"] > 0
    resumed = [s for s in second if s.index in partial and partial[s.index] > 0]
    assert resumed, "buffered groups are served first"
    for s in resumed:
        n_old = partial[s.index]
        assert s.response_length >= n_old and s.loss_mask[:n_old] == [0] * n_old and all(s.loss_mask[n_old:])
        assert len(s.rollout_log_probs) == s.response_length
    m = run.step()          # a full step on top (generation + training) still works with the buffer in place
    assert m["grad_norm"] >= 0
    run.close()
