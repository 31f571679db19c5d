"""Engine pool scale-out / scale-in state machine and the rule-based autoscaler (fake engines, fake clock)."""
import pytest

from relax_b200.rollout.elastic import Autoscaler, AutoscalerConfig, EnginePool, EngineState, Rule
from relax_b200.rollout.router import Router


class _Eng:
    def __init__(self, eid, fail_sync=False):
        self.eid, self.version, self.fail_sync, self.closed, self.aborted = eid, -1, fail_sync, False, False


def _pool(fail_ids=(), clock=None):
    t = clock or [0.0]
    r = Router(clock=lambda: t[0])

    def sync(seed, new):
        if new.fail_sync:
            raise RuntimeError("nvlink copy failed")
        new.version = seed.version
        return new.version

    def abort(e):
        e.aborted = True
        return ["partial-sample"]

    pool = EnginePool(r, lambda eid: _Eng(eid, eid in fail_ids), sync, precheck=lambda s, n: True,
                      shutdown=lambda e: setattr(e, "closed", True), abort=abort, clock=lambda: t[0],
                      sleep=lambda s: t.__setitem__(0, t[0] + s))
    seed = _Eng("seed")
    seed.version = 7
    pool.add_existing("seed", seed, 7)
    return pool, r, t


def test_scale_out_copies_current_weights_and_routes():
    pool, r, _ = _pool()
    res = pool.scale_out(2)
    assert len(res.succeeded) == 2 and not res.failed
    assert all(pool.engines[e].state == EngineState.ACTIVE and pool.engines[e].weight_version == 7 for e in res.succeeded)
    assert set(r.workers()) == {"seed", *res.succeeded}


def test_partial_success_policies():
    pool, r, _ = _pool(fail_ids={"scaled-1"})
    res = pool.scale_out(2, partial_success_policy="keep_partial")
    assert res.succeeded == ["scaled-0"] and "scaled-1" in res.failed
    assert pool.engines["scaled-1"].state == EngineState.FAILED and "scaled-1" not in r.workers()
    pool2, r2, _ = _pool(fail_ids={"scaled-1"})
    res2 = pool2.scale_out(2, partial_success_policy="rollback_all")
    assert res2.rolled_back and not res2.succeeded and set(r2.workers()) == {"seed"}
    assert pool2.engines["scaled-0"].state == EngineState.REMOVED


def test_scale_in_drains_then_aborts_after_timeout():
    pool, r, t = _pool()
    ids = pool.scale_out(2).succeeded
    busy = ids[0]
    # make `busy` hold a request; the other one is idle
    while r.acquire() != busy:
        pass
    for w, st in r.workers().items():
        if w != busy:
            for _ in range(st["in_flight"]):
                r.release(w)
    returned = []
    removed = pool.scale_in(ids=ids, shutdown_timeout_s=1.0, on_abort=returned.extend)
    assert set(removed) == set(ids) and returned == ["partial-sample"]
    assert all(pool.engines[e].state == EngineState.REMOVED for e in ids) and set(r.workers()) == {"seed"}
    assert pool.scale_in(1) == []   # never below min_engines


def test_autoscaler_hold_time_and_cooldowns():
    pool, r, t = _pool()
    m = {"queue_depth_per_engine": 20.0, "kv_cache_utilization": 0.9}
    cfg = AutoscalerConfig(min_engines=1, max_engines=3, scale_out_cooldown_s=100, scale_in_cooldown_s=100,
                           rules=[Rule("queue_depth_per_engine", 8, "above", for_s=30), Rule("kv_cache_utilization", 0.3, "below", for_s=60)])
    a = Autoscaler(pool, cfg, lambda: dict(m), clock=lambda: t[0])
    assert a.step() is None            # condition just started
    t[0] = 31
    assert a.step() == "scale_out" and len(pool.active()) == 2
    t[0] = 70
    assert a.step() is None            # hold time restarts, and cooldown
    t[0] = 140
    assert a.step() == "scale_out" and len(pool.active()) == 3
    t[0] = 300
    assert a.step() is None            # at max_engines
    m.update(queue_depth_per_engine=0.0, kv_cache_utilization=0.1)
    t[0] = 310
    assert a.step() is None
    t[0] = 380
    assert a.step() == "scale_in" and len(pool.active()) == 2
    assert [d[1] for d in a.decisions] == ["scale_out", "scale_out", "scale_in"]
    cfg2 = AutoscalerConfig.from_dict({"max_engines": 4, "rules": [{"metric": "x", "threshold": 1, "direction": "above"}]})
    assert cfg2.max_engines == 4 and cfg2.rules[0].metric == "x"


def test_colocated_loop_recovers_from_engine_failures():
    import pytest
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "8", "--use-health-check",
                    "--rollout-health-check-max-consecutive-failures", "3"])
    c = Controller(a, device="cpu")
    eng = c.runner.engine
    real, calls = eng.generate, {"n": 0, "fail": 2}

    def flaky(*x, **k):                      # the failure is made on the host: the call raises before any work
        calls["n"] += 1
        if calls["n"] <= calls["fail"]:
            raise RuntimeError("engine lost")
        return real(*x, **k)

    eng.generate = flaky
    m = c.runner.step()
    assert calls["n"] == 3 and m["rollout/recoveries"] == 2.0 and m["response_tokens_local"] > 0
    calls.update(n=0, fail=99)
    with pytest.raises(RuntimeError, match="3 times in a row"):
        c.runner.step()


def test_scale_out_and_in_over_real_engines_through_the_control_endpoints():
    """Real engines behind the pool: POST /scale_out creates an engine, copies the seed's CURRENT weights engine to
    engine and admits it (its log-probs equal the seed's), POST /scale_in drains and removes it, GET /engines reports."""
    import json
    import urllib.request

    import torch

    from relax_b200.models.config import get_config
    from relax_b200.rollout.elastic_service import ElasticControlServer, engine_pool
    from relax_b200.rollout.engine import RolloutEngine, SamplingParams

    cfg = get_config("tiny")
    seed = RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=64, block_size=8)
    seed.weights.flat.normal_(0, 0.02, generator=torch.Generator().manual_seed(0))
    seed.update_weight_version(5)
    pool = engine_pool(seed)
    srv = ElasticControlServer(pool)
    base = f"http://{srv.address[0]}:{srv.address[1]}"

    def call(path, body=None):
        req = urllib.request.Request(base + path, data=None if body is None else json.dumps(body).encode(),
                                     method="GET" if body is None else "POST")
        with urllib.request.urlopen(req, timeout=60) as r:
            return json.loads(r.read())

    try:
        out = call("/scale_out", {"num_engines": 2})
        assert len(out["succeeded"]) == 2 and not out["failed"]
        st = call("/engines")
        assert sum(v["state"] == "active" for v in st.values()) == 3 and all(v["weight_version"] == 5 for v in st.values())
        new = pool.engines[out["succeeded"][0]].engine
        assert torch.equal(new.weights.flat, seed.weights.flat) and new.weight_version == 5
        sp = SamplingParams(temperature=0.0, max_new_tokens=5)
        a, b = seed.generate([[3, 4, 5, 6]], sp)[0], new.generate([[3, 4, 5, 6]], sp)[0]
        assert a.output == b.output and a.logprobs == b.logprobs
        assert call("/health")["active"] == 3
        removed = call("/scale_in", {"num_engines": 2})["removed"]
        assert len(removed) == 2 and "seed" not in removed and len(pool.active()) == 1
        import urllib.error

        with pytest.raises(urllib.error.HTTPError) as bad:       # a bad request is answered with 400, the service lives on
            call("/scale_out", {"num_engines": 1, "policy": "nonsense"})
        assert bad.value.code == 400 and call("/health")["status"] == "ok"
    finally:
        srv.close()


def test_elastic_pool_of_external_engine_servers_in_a_training_job(tmp_path):
    """A training job on one pre-launched engine server grows to three while it runs: a scale-out request by URL (the
    new server gets the CURRENT weights before it sees a request; repeating the request is a no-op), a second server
    brought in by an autoscaling rule from the standby list, then a scale-in that drains one and leaves it running."""
    import json
    import time
    import urllib.request

    import torch

    from relax_b200.config.arguments import parse_args
    from relax_b200.models.config import get_config
    from relax_b200.orchestration.controller import Controller
    from relax_b200.rollout.engine import RolloutEngine
    from relax_b200.rollout.http_server import EngineServer, HTTPEngine

    cfg = get_config("tiny")
    servers = [EngineServer(RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=128, block_size=8, seed=i)) for i in range(3)]
    addr = [s.url.replace("http://", "") for s in servers]
    rules = tmp_path / "rules.json"
    rules.write_text(json.dumps({"min_engines": 1, "max_engines": 3, "scale_out_cooldown_s": 0.0, "scale_in_cooldown_s": 1e9,
                                 "rules": [{"metric": "num_engines", "threshold": 2.5, "direction": "below", "for_s": 1e9},
                                           {"metric": "always_high", "threshold": 0.5, "direction": "above", "for_s": 0.0}]}))

    def call(url, path, body=None):
        req = urllib.request.Request(url + path, data=None if body is None else json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=60) as r:
            return json.loads(r.read())

    try:
        a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2",
                        "--global-batch-size", "8", "--num-rollout", "3", "--rollout-max-response-len", "5", "--rollout-max-prompt-len", "16",
                        "--lr", "1e-2", "--rm-type", "token_sum_parity", "--rollout-external", "--rollout-external-engine-addrs", addr[0],
                        "--elastic-control-port", "0", "--autoscaler-config", str(rules), "--autoscaler-interval", "1000",
                        "--rollout-standby-engine-addrs", addr[2], "--scale-weight-sync-precheck", "--scale-out-timeout", "60"])
        c = Controller(a, device="cpu")
        run = c.runner
        ctl = f"http://127.0.0.1:{run.elastic.address[1]}"
        run.step()
        v1 = run.actor.weight_version
        assert servers[0].engine.weight_version == v1 and servers[1].engine.weight_version == 0
        # scale out by URL: accepted, runs in the background, the server ends up ACTIVE with the current weights
        out = call(ctl, "/scale_out", {"engine_urls": [addr[1]], "timeout_secs": 60})
        assert out["status"] == "PENDING"
        deadline = time.monotonic() + 60
        while call(ctl, "/scale_out")["requests"][-1]["status"] in ("PENDING", "SYNCING") and time.monotonic() < deadline:
            time.sleep(0.05)
        last = call(ctl, "/scale_out?status=ACTIVE")["requests"]
        assert len(last) == 1 and last[0]["succeeded"] == [servers[1].url]
        assert servers[1].engine.weight_version == v1
        assert all(torch.equal(servers[1].engine.weights.p[k], servers[0].engine.weights.p[k]) for k in servers[0].engine.weights.p)
        assert call(ctl, "/scale_out", {"engine_urls": [addr[1]]})["status"] == "NOOP"
        served = servers[1].served
        m = run.step()                                             # both servers generate and take the next weights
        assert m["rollout/engines_active"] == 2.0 and servers[1].served > served
        assert servers[1].engine.weight_version == servers[0].engine.weight_version == run.actor.weight_version == v1 + 1
        # the autoscaler brings in the standby server
        run.elastic.autoscaler.metrics_fn = lambda: dict(run.engine.server_metrics(), always_high=1.0)
        assert call(ctl, "/autoscale_step", {})["action"] == "scale_out"
        assert len(run.elastic.pool.active()) == 3 and servers[2].engine.weight_version == v1 + 1
        # scale in by URL: drained, forgotten, still running
        assert call(ctl, "/scale_in", {"engine_urls": [addr[1]], "timeout": 5})["removed"] == [servers[1].url]
        served = servers[1].served
        m = run.step()
        assert m["rollout/engines_active"] == 2.0 and servers[1].served == served and HTTPEngine(servers[1].url).health()
        assert servers[1].engine.weight_version == v1 + 1 and servers[2].engine.weight_version == v1 + 2
        eng = call(ctl, "/engines")
        assert eng[servers[1].url]["state"] == "removed" and eng[servers[2].url]["state"] == "active"
        # what a Prometheus scraper sees: pool gauges on the control port, engine gauges on every server
        text = urllib.request.urlopen(ctl + "/metrics", timeout=10).read().decode()
        assert "relax_rollout_engines_active 2" in text and "relax_rollout_autoscaler_decisions_total 1" in text
        text = urllib.request.urlopen(servers[0].url + "/metrics", timeout=10).read().decode()
        assert "# TYPE relax_engine_kv_cache_usage gauge" in text and f"relax_engine_weight_version {v1 + 2}" in text
        assert "relax_engine_requests_served_total" in text
        run.close()
    finally:
        for s in servers:
            s.close()
