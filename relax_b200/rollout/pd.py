"""Prefill / decode disaggregation: prompts are prefilled on one engine, their KV cache moves, decoding goes on elsewhere.

Prefill is compute-bound and bursty, decode is bound by reading the weights and steady; on one engine every prefill
stalls the running decode batch for its whole length.  Serving stacks therefore run the two phases on different
engines and ship the prompt's KV cache between them - the reference configures its engines that way with
``--prefill-num-servers`` (relax/distributed/ray/rollout.py:139 ``has_pd_disaggregation``, :202
``SglangConfig.from_prefill_num_servers``: prefill and decode worker groups behind a PD-aware router, a bootstrap port
per engine for the KV transfer :4153).

Here the hand-over is explicit and small:

* :func:`detach` takes requests that just finished their prefill out of an engine: token state plus the contents of
  their KV blocks, gathered into one contiguous tensor ``[layers, 2, tokens, kv_heads, head_dim]`` (block size and
  block ids are private to an engine); the blocks go back to the prefill engine at once.
* :func:`attach` gives such a request to another engine: blocks are allocated there for the request's whole maximum
  length, the KV rows are scattered into them, and the request joins the running batch as if it had been prefilled
  locally - its first token (sampled by the prefill engine) is already in ``output``.
* :class:`PDEngine` is the pair behind the engine's ``generate`` signature.  ``transfer`` is the wire: identity for
  two engines on one device, ``PeerTransfer`` for engines on two ranks (KV tensor by point-to-point send/recv, the
  rest as a small object).

The engines must serve the same model with the same tensor-parallel degree (the KV heads of a rank travel to the rank
with the same index).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from .engine import Request, RolloutEngine, SamplingParams


@dataclass
class PrefilledRequest:
    prompt: list
    output: list
    logprobs: list
    weight_versions: list
    params: SamplingParams
    group_key: Optional[int]
    pos_delta: int
    kv: torch.Tensor                       # [layers, 2, tokens fed so far, kv_heads, head_dim]
    tag: object = None                     # the caller's handle (e.g. the index of the prompt)
    status: str = "running"
    finish_reason: Optional[str] = None
    cached_tokens: int = 0
    times: dict = field(default_factory=dict)


def detach(engine: RolloutEngine, reqs: Sequence[Request]) -> List[PrefilledRequest]:
    """Take ``reqs`` (running on ``engine``, prefilled) out of it together with their KV rows; frees their blocks."""
    if getattr(engine, "hybrid", False):
        raise NotImplementedError("the hand-over moves paged K/V; the recurrent state of Gated-DeltaNet layers does not travel yet")
    out = []
    bs = engine.block_size
    for r in reqs:
        n = r.num_tokens - 1                  # the newest token has not been fed yet
        idx = torch.tensor([r.blocks[p // bs] * bs + p % bs for p in range(n)], dtype=torch.long, device=engine.kv.device)
        L, two, nb, _, hkv, hd = engine.kv.shape
        kv = engine.kv.view(L, two, nb * bs, hkv, hd).index_select(2, idx).contiguous()
        out.append(PrefilledRequest(list(r.prompt), list(r.output), list(r.logprobs), list(r.weight_versions), r.params, r.group_key,
                                    r.pos_delta, kv, status=r.status, finish_reason=r.finish_reason, cached_tokens=r.cached_tokens,
                                    times={"t_arrive": r.t_arrive, "t_first": r.t_first}))
        engine.bm.release(r.blocks)
        r.blocks, r._reserve = [], 0
    gone = {id(r) for r in reqs}
    engine.running = [r for r in engine.running if id(r) not in gone]
    return out


def can_attach(engine: RolloutEngine, p: PrefilledRequest) -> bool:
    need = engine.bm.blocks_for(len(p.prompt) + p.params.max_new_tokens)
    reserved = sum(getattr(x, "_reserve", 0) for x in engine.running)
    return len(engine.running) < engine.max_running and need <= engine.bm.num_free - reserved


def attach(engine: RolloutEngine, p: PrefilledRequest) -> Request:
    """Continue ``p`` on ``engine``: blocks, KV rows, a running request.  Call :func:`can_attach` first."""
    L, two, n, hkv, hd = p.kv.shape
    eL = engine.kv.shape[0]
    if (eL, engine.kv.shape[4], engine.kv.shape[5]) != (L, hkv, hd):
        raise ValueError(f"KV layout differs: {tuple(p.kv.shape)} does not fit an engine with {tuple(engine.kv.shape)}")
    r = Request(engine._next_rid, list(p.prompt), p.params, p.group_key, output=list(p.output), logprobs=list(p.logprobs),
                weight_versions=list(p.weight_versions), status="running", cached_tokens=p.cached_tokens, pos_delta=p.pos_delta,
                t_arrive=p.times.get("t_arrive", 0.0), t_first=p.times.get("t_first", 0.0))
    engine._next_rid += 1
    bs = engine.block_size
    need_total = engine.bm.blocks_for(len(r.prompt) + r.params.max_new_tokens)
    nb = engine.bm.blocks_for(r.num_tokens)
    r.blocks = [engine.bm.alloc() for _ in range(nb)]
    r._reserve, r._lead = need_total - nb, None
    idx = torch.tensor([r.blocks[q // bs] * bs + q % bs for q in range(n)], dtype=torch.long, device=engine.kv.device)
    _, _, enb, _, _, _ = engine.kv.shape
    engine.kv.view(L, two, enb * bs, hkv, hd).index_copy_(2, idx, p.kv.to(device=engine.kv.device, dtype=engine.kv.dtype))
    engine.running.append(r)
    return r


class PeerTransfer:
    """The wire between a prefill rank and a decode rank: metadata as an object, the KV tensor point to point."""

    def __init__(self, src: int, dst: int, group=None, device="cpu", dtype=torch.float32):
        self.src, self.dst, self.group, self.device, self.dtype = src, dst, group, device, dtype

    def send(self, items: List[PrefilledRequest]):
        import torch.distributed as dist

        meta = [(p.prompt, p.output, p.logprobs, p.weight_versions, p.params, p.group_key, p.pos_delta, tuple(p.kv.shape), p.tag,
                 p.status, p.finish_reason, p.cached_tokens, p.times) for p in items]
        dist.send_object_list([meta], dst=self.dst, group=self.group)
        for p in items:
            dist.send(p.kv.contiguous(), dst=self.dst, group=self.group)

    def recv(self) -> List[PrefilledRequest]:
        import torch.distributed as dist

        box = [None]
        dist.recv_object_list(box, src=self.src, group=self.group)
        out = []
        for (prompt, output, lps, wv, params, key, delta, shape, tag, status, reason, cached, times) in box[0]:
            kv = torch.empty(shape, dtype=self.dtype, device=self.device)
            dist.recv(kv, src=self.src, group=self.group)
            out.append(PrefilledRequest(prompt, output, lps, wv, params, key, delta, kv, tag, status, reason, cached, times))
        return out


class PDEngine:
    """A prefill engine and a decode engine behind ``generate``.  Both in this process (the same or different devices);
    ``stats`` counts the hand-overs and the KV bytes moved."""

    def __init__(self, prefill: RolloutEngine, decode: RolloutEngine, transfer: Optional[Callable] = None):
        if prefill.cfg.name != decode.cfg.name or prefill.tp.size != decode.tp.size:
            raise ValueError("prefill and decode engines must serve the same model with the same tensor-parallel degree")
        self.prefill, self.decode = prefill, decode
        self.transfer = transfer or (lambda items: items)
        self.cfg, self.device = decode.cfg, decode.device
        self.stats = {"handed_over": 0, "kv_bytes": 0, "prefill_steps": 0, "decode_steps": 0}

    @property
    def weight_version(self) -> int:
        return self.decode.weight_version

    def generate(self, prompts: Sequence[Sequence[int]], params, group_keys: Optional[Sequence] = None, images=None):
        if images is not None and any(images):
            raise NotImplementedError("image prompts are prefilled and decoded on one engine")
        pe, de = self.prefill, self.decode
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        tag_of = {}
        for i, (p, sp) in enumerate(zip(prompts, plist)):
            rid = pe.add_request(p, sp, group_keys[i] if group_keys is not None else None)
            tag_of[rid] = i
        results: dict = {}
        parked: List[PrefilledRequest] = []         # prefilled, waiting for room on the decode engine
        owner: dict = {}                            # decode request id -> prompt index
        while pe.has_work or parked or de.has_work:
            if pe.waiting:
                before = len(pe.waiting)
                done = pe.step()                    # admits and prefills; nothing is decoded here
                self.stats["prefill_steps"] += 1
                if len(pe.waiting) == before and not done and not pe.running:
                    raise RuntimeError("the prefill engine cannot admit the next prompt: its KV cache is too small for it")
                for r in done:                      # finished with its first token (stop token, max_new_tokens = 1)
                    results[tag_of[r.rid]] = r
                fresh = list(pe.running)
                if fresh:
                    items = detach(pe, fresh)
                    for r, it in zip(fresh, items):
                        it.tag = tag_of[r.rid]
                    items = self.transfer(items)
                    self.stats["handed_over"] += len(items)
                    self.stats["kv_bytes"] += sum(it.kv.numel() * it.kv.element_size() for it in items)
                    parked += items
            while parked and can_attach(de, parked[0]):
                it = parked.pop(0)
                owner[attach(de, it).rid] = it.tag
            if de.running:
                for r in de.step():
                    results[owner.pop(r.rid)] = r
                self.stats["decode_steps"] += 1
            elif parked and not pe.waiting:
                raise RuntimeError("the decode engine cannot take a prefilled request: its KV cache is too small for it")
        return [results[i] for i in range(len(prompts))]

    # the parts of the engine surface that weight sync and the loops use
    def pause_generation(self):
        self.prefill.pause_generation()
        self.decode.pause_generation()

    def continue_generation(self):
        self.prefill.continue_generation()
        self.decode.continue_generation()

    def flush_cache(self):
        self.prefill.flush_cache()
        self.decode.flush_cache()

    def update_weight_version(self, v: int):
        self.prefill.update_weight_version(v)
        self.decode.update_weight_version(v)

    def close(self):
        self.prefill.close()
        self.decode.close()
