"""Router (least-loaded, sticky, health, drain) and the text radix cache."""
import pytest

from relax_b200.rollout.radix_cache import RadixCache
from relax_b200.rollout.router import NoHealthyWorker, Router


def test_least_loaded_and_sticky():
    t = [0.0]
    r = Router(sticky_idle_s=10, clock=lambda: t[0])
    for w in "abc":
        r.add_worker(w)
    first = r.acquire("group-1")
    # same key keeps its worker even though it is now the most loaded
    assert r.acquire("group-1") == first
    others = {r.acquire(), r.acquire()}
    assert first not in others and len(others) == 2
    r.release(first)
    r.release(first)
    t[0] = 100.0   # sticky entry expired: falls back to least loaded
    nxt = r.acquire("group-1")
    assert nxt == first   # idle again, fewest in flight
    assert r.workers()[first]["in_flight"] == 1


def test_quarantine_readmit_and_drain():
    r = Router(max_failures=2)
    r.add_worker("a")
    r.add_worker("b")
    alive = {"a": True, "b": False}
    r.check_health(lambda h: alive[h])
    assert r.workers()["b"]["healthy"]
    r.check_health(lambda h: alive[h])
    assert not r.workers()["b"]["healthy"]
    assert {r.acquire() for _ in range(4)} == {"a"}
    alive["b"] = True
    r.check_health(lambda h: alive[h])
    assert r.workers()["b"]["healthy"]
    r.drain_worker("a")
    assert r.acquire() == "b"
    assert not r.is_idle("a")
    for _ in range(4):
        r.release("a")
    assert r.is_idle("a")
    r.remove_worker("a")
    r.release("b", failed=True)
    r.release("b", failed=True)
    with pytest.raises(NoHealthyWorker):
        r.acquire()


def _tok(s):
    return [ord(c) for c in s]


def test_radix_prefix_reuse_and_versions():
    c = RadixCache(tokenizer=_tok, gc_threshold_k=2)
    p = "system: be brief\nuser: hi\n"
    c.insert(p, _tok(p), weight_version=1)
    turn1 = p + "assistant: hello\n"
    gen = _tok("assistant: hello\n")
    c.insert(turn1, _tok(p) + gen, [0.0] * len(p) + [-0.5] * len(gen), [0] * len(p) + [1] * len(gen), weight_version=1)
    m = c.find_longest_prefix(turn1 + "user: more\n")
    assert m.matched_prefix == turn1 and m.remaining == "user: more\n"
    assert m.token_ids == _tok(turn1) and sum(m.loss_mask) == len(gen) and m.logp[-1] == -0.5
    toks, lps, mask = c.retrieve_from_text(turn1 + "user: more\n")
    assert toks == _tok(turn1 + "user: more\n") and mask[-1] == 0
    assert c.stats()["tokens"] == len(toks)
    # mismatching tokens for a cached prefix are rejected
    with pytest.raises(ValueError):
        c.insert(turn1 + "x", [1, 2, 3])
    # a branch written by old weights is collected, the refreshed one stays
    other = p + "assistant: bye\n"
    c.insert(other, _tok(other), weight_version=1)
    c.insert(turn1, _tok(turn1), weight_version=5)   # touch: refreshes versions along the path
    freed = c.gc_by_weight_version(5)
    assert freed > 0
    assert c.find_longest_prefix(other).matched_prefix == p
    assert c.find_longest_prefix(turn1).matched_prefix == turn1


def test_radix_lru_eviction():
    c = RadixCache(max_tokens=30)
    c.insert("aaaaaaaaaa", list(range(10)))
    c.insert("bbbbbbbbbb", list(range(10)))
    c.find_longest_prefix("aaaaaaaaaa")   # refresh a
    c.insert("cccccccccccccccc", list(range(16)))
    assert c.stats()["tokens"] <= 30
    assert c.find_longest_prefix("bbbbbbbbbb").matched_prefix == ""
    assert c.find_longest_prefix("aaaaaaaaaa").matched_prefix == "aaaaaaaaaa"


def test_http_router_proxies_sticks_and_fails_over():
    """The router as an HTTP proxy: requests go to registered workers (least loaded, sticky by session), a dead
    worker is skipped after a failed attempt, membership changes over HTTP."""
    import json
    import threading
    import urllib.request
    from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

    from relax_b200.rollout.router import Router, serve_router

    def upstream(tag):
        class H(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def do_GET(self):
                self.send_response(200); self.end_headers(); self.wfile.write(b"{}")

            def do_POST(self):
                n = int(self.headers.get("Content-Length", "0"))
                body = json.loads(self.rfile.read(n) or b"{}")
                out = json.dumps({"worker": tag, "echo": body.get("text")}).encode()
                self.send_response(200); self.send_header("Content-Length", str(len(out))); self.end_headers(); self.wfile.write(out)
        s = ThreadingHTTPServer(("127.0.0.1", 0), H)
        threading.Thread(target=s.serve_forever, daemon=True).start()
        return s, f"http://127.0.0.1:{s.server_address[1]}"

    a, ua = upstream("a")
    b, ub = upstream("b")
    srv, _, router = serve_router(Router(max_failures=1), health_interval_s=0)
    base = f"http://127.0.0.1:{srv.server_address[1]}"

    def post(path, obj):
        req = urllib.request.Request(base + path, data=json.dumps(obj).encode(), headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=10) as r:
            return json.loads(r.read())

    post("/add_worker", {"url": ua})
    post("/add_worker?url=" + ub, {})
    with urllib.request.urlopen(base + "/list_workers") as r:
        assert sorted(json.loads(r.read())["urls"]) == sorted([ua, ub])
    first = post("/generate", {"text": "x", "session_id": "s1"})["worker"]
    assert all(post("/generate", {"text": "y", "session_id": "s1"})["worker"] == first for _ in range(4))     # sticky
    seen = {post("/generate", {"text": str(i)})["worker"] for i in range(6)}
    assert seen == {"a", "b"}
    # kill one upstream: its requests fail over to the other and it is quarantined
    (a if first == "a" else b).shutdown()
    (a if first == "a" else b).server_close()
    other = "b" if first == "a" else "a"
    assert all(post("/generate", {"text": "z", "session_id": "s1"})["worker"] == other for _ in range(3))
    post("/remove_worker", {"url": ua if first == "a" else ub})
    with urllib.request.urlopen(base + "/list_workers") as r:
        assert len(json.loads(r.read())["urls"]) == 1
    srv.shutdown(); srv.server_close(); router.stop()
    (b if first == "a" else a).shutdown()


def test_engine_http_server_behind_the_router_matches_in_process_generation():
    """Two engine servers (same weights, same seed) behind the HTTP router: greedy generations through the proxy equal
    the in-process engine's, concurrent requests are batched, control routes work."""
    import json
    import threading
    import urllib.request

    import torch

    from relax_b200.models.config import get_config
    from relax_b200.rollout.engine import RolloutEngine, SamplingParams
    from relax_b200.rollout.http_server import EngineServer, HTTPEngine
    from relax_b200.rollout.router import Router, serve_router
    from relax_b200.train.actor import TrainActor, TrainConfig
    from relax_b200.weight_sync.plan import TrainerLayout
    from relax_b200.weight_sync.sync import WeightSync

    cfg = get_config("tiny")
    actor = TrainActor(cfg, TrainConfig(), seed=0, with_optimizer=False)

    def engine():
        e = RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=128, block_size=8)
        WeightSync(cfg, TrainerLayout(), 1, [0], [0]).update_weights(dict(actor.named_local_params()), e.weights, e, 1)
        return e

    local = engine()
    servers = [EngineServer(engine()), EngineServer(engine())]
    srv, _, router = serve_router(Router(), health_interval_s=0)
    for s in servers:
        router.add_worker(s.url)
    base = f"http://127.0.0.1:{srv.server_address[1]}"
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (6, 9, 5, 12)]
    sp = SamplingParams(max_new_tokens=7, temperature=1.0, top_k=1)       # greedy: comparable across engines
    want = local.generate(prompts, sp)
    got = HTTPEngine(base).generate(prompts, sp)
    for a, b in zip(got, want):
        assert a.output == b.output and max(abs(x - y) for x, y in zip(a.logprobs, b.logprobs)) < 1e-5
    # concurrent single-prompt requests are spread over the workers and all answered
    outs = [None] * 4

    def one(i):
        outs[i] = HTTPEngine(base).generate([prompts[i]], sp)[0].output

    ts = [threading.Thread(target=one, args=(i,)) for i in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert outs == [w.output for w in want]
    assert sum(s.served for s in servers) == 8 and all(s.served > 0 for s in servers)
    with urllib.request.urlopen(servers[0].url + "/get_server_info") as r:
        info = json.loads(r.read())
    assert info["weight_version"] == 1 and info["running"] == 0
    assert HTTPEngine(servers[0].url).flush_cache()["status"] == "ok"
    for s in servers:
        s.close()
    srv.shutdown(); srv.server_close(); router.stop()


def test_external_engines_driven_by_the_colocated_loop():
    """``--rollout-external``: two pre-launched engine servers; the training job checks what they serve, generates
    through them and ships its weights after every step.  The servers end up with the trainer's weights, bit for
    bit, and are still running when the job is gone."""
    import torch

    from relax_b200.config.arguments import parse_args
    from relax_b200.models.config import get_config
    from relax_b200.orchestration.controller import Controller
    from relax_b200.rollout.engine import RolloutEngine
    from relax_b200.rollout.http_server import EngineServer, HTTPEngine
    from relax_b200.weight_sync.sync import oracle_rollout_state

    cfg = get_config("tiny")
    servers = [EngineServer(RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=128, block_size=8, seed=7 + i))
               for i in range(2)]
    try:
        addrs = [s.url.replace("http://", "") for s in servers]
        with pytest.raises(ValueError, match="engine-addrs"):
            parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "4", "--rollout-external"])
        a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "4", "--n-samples-per-prompt", "2",
                        "--global-batch-size", "8", "--num-rollout", "2", "--rollout-max-response-len", "6", "--rollout-max-prompt-len", "16",
                        "--lr", "1e-2", "--rm-type", "token_sum_parity", "--rollout-external", "--rollout-external-engine-addrs", *addrs])
        c = Controller(a, device="cpu")
        assert all(s.engine.weight_version == c.runner.actor.weight_version for s in servers)      # initial sync reached them
        before = {k: v.clone() for k, v in servers[0].engine.weights.p.items()}
        for _ in range(2):
            m = c.runner.step()
        assert m["response_tokens_local"] > 0 and all(s.served > 0 for s in servers)              # both servers generated
        want = oracle_rollout_state(cfg, dict(c.runner.actor.named_local_params()), 1, 0)
        for s in servers:
            assert s.engine.weight_version == c.runner.actor.weight_version == 2
            for k, w in want.items():
                assert torch.equal(s.engine.weights.p[k], w.to(s.engine.weights.p[k].dtype)), k
        assert any(not torch.equal(before[k], servers[0].engine.weights.p[k]) for k in before)
        c.runner.close()
        assert HTTPEngine(servers[0].url).health()                                                  # not ours to stop
        # a server that serves another model is refused at start-up
        other = EngineServer(RolloutEngine(get_config("tiny-moe"), device="cpu", dtype=torch.float32, num_kv_blocks=32, block_size=8))
        try:
            a2 = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "4", "--rollout-external",
                             "--rollout-external-engine-addrs", other.url.replace("http://", "")])
            with pytest.raises(ValueError, match="serves model"):
                Controller(a2, device="cpu")
        finally:
            other.close()
    finally:
        for s in servers:
            s.close()


def test_external_engine_fails_over_when_a_server_dies():
    """A server that stops answering in the middle of a job: its prompt groups are generated by the other one, the dead
    server is out of rotation, and weight updates report the failure instead of hanging."""
    import torch

    from relax_b200.models.config import get_config
    from relax_b200.rollout.engine import RolloutEngine, SamplingParams
    from relax_b200.rollout.external import ExternalEngine
    from relax_b200.rollout.http_server import EngineServer
    from relax_b200.rollout.router import NoHealthyWorker

    cfg = get_config("tiny")
    servers = [EngineServer(RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=128, block_size=8, seed=i)) for i in range(2)]
    try:
        ext = ExternalEngine(cfg, [s.url for s in servers], "cpu", torch.float32, timeout_s=20.0)
        prompts = [[5 + i, 6, 7, 8] for i in range(6)]
        sp = SamplingParams(temperature=0.0, max_new_tokens=4)
        first = ext.generate(prompts, sp, group_keys=list(range(6)))
        assert all(len(r.output) == 4 for r in first) and all(s.served > 0 for s in servers)
        servers[1].close()
        again = ext.generate(prompts, sp, group_keys=list(range(10, 16)))
        assert all(len(r.output) == 4 for r in again) and ext.stats["failovers"] >= 1
        w = ext.router.workers()
        assert w[servers[1].url]["healthy"] is False and w[servers[0].url]["healthy"] is True
        third = ext.generate(prompts, sp, group_keys=list(range(20, 26)))          # no request reaches the dead server any more
        assert all(len(r.output) == 4 for r in third)
        # weight updates go to the servers in rotation only; a replacement on the same address is brought up to date
        # before it gets requests again
        with torch.no_grad():
            for t in ext.weights.p.values():
                t.fill_(0.01)
        ext.update_weight_version(5)
        assert servers[0].engine.weight_version == 5
        port = int(servers[1].url.rsplit(":", 1)[1])
        servers[1] = EngineServer(RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=128, block_size=8, seed=9), port=port)
        fourth = ext.generate(prompts, sp, group_keys=list(range(30, 36)))
        assert all(len(r.output) == 4 for r in fourth) and ext.router.workers()[servers[1].url]["healthy"]
        assert servers[1].engine.weight_version == 5 and float(servers[1].engine.weights.p["final_norm"][0]) == pytest.approx(0.01)
        servers[1].close()
        servers[0].close()
        with pytest.raises((NoHealthyWorker, RuntimeError)):
            ext.generate(prompts[:1], sp)
        ext.close()
    finally:
        for s in servers:
            try:
                s.close()
            except Exception:  # noqa: BLE001 - already closed above
                pass
