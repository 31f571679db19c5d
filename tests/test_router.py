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
