"""In-house rollout (inference) engine: paged KV cache, continuous batching,
group prefix sharing, sampling with log-prob return, abort / partial rollout,
weight-version tagging and tagged memory release.

It fills the place the reference gives to an external inference server
(relax/backends/sglang/sglang_engine.py:339-1450; request fields used by
relax/engine/rollout/sglang_rollout.py:299-493: ``input_ids``, sampling
params, ``return_logprob``).  One engine spans a tensor-parallel group of
rollout ranks; all ranks of the group run the same scheduler deterministically
(same requests, same random draws), so no control messages cross ranks inside
the decode loop - only the collectives inside the model.
"""
from __future__ import annotations

import math
import os
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .. import ops
from ..models.config import ModelConfig
from ..parallel.state import GroupInfo
from .speculative import SpeculativeMixin
from .weights import RolloutWeights


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    max_new_tokens: int = 1024
    stop_token_ids: tuple = ()
    ignore_eos: bool = False
    no_stop_trim: bool = False


@dataclass
class Request:
    rid: int
    prompt: list
    params: SamplingParams
    group_key: Optional[int] = None
    output: list = field(default_factory=list)
    logprobs: list = field(default_factory=list)
    blocks: list = field(default_factory=list)
    status: str = "waiting"        # waiting | running | finished | aborted
    finish_reason: Optional[str] = None
    weight_versions: list = field(default_factory=list)
    cached_tokens: int = 0
    # with ``return_routed_experts``: per context position that was fed to the model, the expert ids every MoE layer
    # chose - a list of ``[L_moe, k]`` int lists (positions 0 .. num_tokens - 2; the last token is never fed)
    routed_experts: list = field(default_factory=list)
    # multimodal prompts: pre-cut patches of the prompt's images (``[N, patch_dim]`` + ``grid_thw [n_img, 3]``) or
    # their embeddings (``[n_image_tokens, hidden]``), the M-RoPE position ids of the prompt ``[3][len(prompt)]`` and
    # the offset between a generated token's index in the sequence and its rotary position
    pixel_patches: Optional[torch.Tensor] = None
    grid_thw: Optional[torch.Tensor] = None
    image_embeds: Optional[torch.Tensor] = None
    mrope_positions: Optional[list] = None
    pos_delta: int = 0
    t_arrive: float = 0.0
    t_first: float = 0.0
    t_done: float = 0.0
    # speculative decoding: proposals checked / accepted and verify passes of this request
    spec_draft: int = 0
    spec_accept: int = 0
    spec_verify: int = 0

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)


class BlockManager:
    """Reference-counted fixed-size KV blocks."""

    def __init__(self, num_blocks: int, block_size: int):
        self.num_blocks, self.block_size = num_blocks, block_size
        self.free = deque(range(num_blocks))
        self.ref = [0] * num_blocks

    @property
    def num_free(self) -> int:
        return len(self.free)

    def alloc(self) -> int:
        if not self.free:
            raise RuntimeError("KV cache exhausted")
        b = self.free.popleft()
        self.ref[b] = 1
        return b

    def share(self, b: int) -> int:
        self.ref[b] += 1
        return b

    def release(self, blocks: Sequence[int]):
        for b in blocks:
            self.ref[b] -= 1
            if self.ref[b] == 0:
                self.free.append(b)
            elif self.ref[b] < 0:
                raise RuntimeError(f"block {b} released twice")

    def blocks_for(self, ntokens: int) -> int:
        return (ntokens + self.block_size - 1) // self.block_size


class RolloutEngine(SpeculativeMixin):
    def __init__(self, cfg: ModelConfig, tp: Optional[GroupInfo] = None, device="cpu", dtype=None,
                 num_kv_blocks: int = 256, block_size: int = 16, max_running: int = 256,
                 max_prefill_tokens: int = 16384, seed: int = 42, eos_token_id: Optional[int] = None,
                 use_cuda_graph: bool = True, max_model_len: int = 4096, memory_saver: Optional[bool] = None,
                 decode_window: Optional[int] = None, windowed_decode: Optional[bool] = None,
                 weights_shared_path: Optional[str] = None, ep: Optional[GroupInfo] = None,
                 return_routed_experts: bool = False, speculative: bool = False, speculative_steps: int = 1):
        self.cfg = cfg
        # speculative decoding drafted by the model's multi-token-prediction block (rollout/speculative.py)
        self.speculative = bool(speculative)
        self.speculative_steps = max(1, int(speculative_steps))      # proposals per verify pass (the block is chained)
        if self.speculative:
            if cfg.mtp_num_layers < 1:
                raise ValueError("speculative decoding drafts with the model's multi-token-prediction block; this model has none")
            if cfg.vision is not None or (return_routed_experts and cfg.is_moe) or cfg.linear_attention_freq > 0:
                raise NotImplementedError("speculative decoding serves text prompts of softmax-attention models and does not "
                                          "record routed experts")
        self.tp = tp or GroupInfo(None, (0,), 0)
        self.device = torch.device(device)
        self.dtype = dtype or {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[cfg.dtype]
        # pausable buffers keep their addresses across release/resume, so CUDA graphs survive the trainer's turn
        if memory_saver is None:
            memory_saver = self.device.type == "cuda" and os.environ.get("RELAX_B200_MEMORY_SAVER", "1") == "1"
        self.memory_saver = bool(memory_saver)
        self._kv_buf = None
        # expert parallelism inside one engine: every rank of ``ep`` runs the whole batch (attention replicated),
        # holds ``num_experts / ep`` experts and the experts' partial outputs are summed over the group
        self.ep = ep if (ep is not None and ep.size > 1) else None
        if self.ep is not None and self.tp.size > 1:
            raise NotImplementedError("an engine is tensor-parallel or expert-parallel, not both")
        self.weights = RolloutWeights(cfg, self.tp.size, self.tp.rank, self.device, self.dtype,
                                      ep_size=self.ep.size if self.ep else 1, ep_rank=self.ep.rank if self.ep else 0,
                                      memory_saver=self.memory_saver, shared_path=weights_shared_path, mtp=self.speculative)
        self.weights.ep_group = self.ep
        self.return_routed_experts = bool(return_routed_experts) and cfg.is_moe
        self.block_size = block_size
        self.bm = BlockManager(num_kv_blocks, block_size)
        self.max_running, self.max_prefill_tokens = max_running, max_prefill_tokens
        self.eos = eos_token_id
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self._next_rid = 0
        self.paused = False
        self.weight_version = 0
        self.gen = torch.Generator(device="cpu").manual_seed(seed)
        self.kv = None
        self._alloc_kv()
        self.use_cuda_graph = use_cuda_graph and self.device.type == "cuda"
        self.max_model_len = max_model_len
        # decode steps issued back to back between two host synchronisations: the batch state (tokens, positions,
        # context lengths, cache slots) is advanced on the device, the host reads the sampled tokens once per window
        if decode_window is None:
            decode_window = int(os.environ.get("RELAX_B200_DECODE_WINDOW", "16"))
        self.decode_window = max(1, int(decode_window))
        self.windowed_decode = self.use_cuda_graph if windowed_decode is None else bool(windowed_decode)
        if self.speculative:
            self.windowed_decode = False     # the rows per request change from step to step: host-driven iterations
        # hybrid stacks: Gated-DeltaNet layers keep a convolution window and a recurrent matrix per request
        # (Request._gdn: layer -> [window, matrix]) next to the paged K/V of the softmax layers; host-driven decode
        self.hybrid = cfg.linear_attention_freq > 0 or cfg.dsa_topk > 0 or cfg.multi_latent_attention
        # latent-attention layers (MLA / DSA) keep per request the latent rows (and indexer keys) of every fed token
        # (Request._mla: layer -> [rows, keys]), pre-sized for the request's maximum length
        self.latent = cfg.dsa_topk > 0 or cfg.multi_latent_attention
        if self.hybrid:
            self.windowed_decode = False
            self.use_cuda_graph = False
        if os.environ.get("RELAX_B200_FORCE_REFERENCE", "0") == "1" and self.device.type == "cuda":
            self.windowed_decode = False     # the library-path arm keeps the host-driven loop
        self._graphs = {}
        self._graph_pool = None
        # padding rows of a graph bucket read/write this block; it is never handed to a request
        self._scratch_block = self.bm.alloc() if (self.use_cuda_graph or self.windowed_decode) else 0
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "cached_tokens": 0, "steps": 0}

    # ------------------------------------------------------------------ memory
    def _alloc_kv(self):
        c = self.cfg
        hkv = c.num_query_groups // self.tp.size
        # with speculative decoding the draft block keeps its own cache as one more layer under the same block tables
        shape = (c.num_layers + (1 if self.speculative else 0), 2, self.bm.num_blocks, self.block_size, hkv, c.head_dim)
        if self.memory_saver:
            from ..utils.memory_saver import PausableBuffer

            if self._kv_buf is None:
                self._kv_buf = PausableBuffer(math.prod(shape) * torch.empty(0, dtype=self.dtype).element_size(), self.device)
                self.kv = self._kv_buf.tensor(shape, self.dtype)
            else:
                self._kv_buf.resume()
            return
        self.kv = torch.zeros(*shape, dtype=self.dtype, device=self.device)

    def release_memory_occupation(self, tags: Sequence[str] = ("kv_cache", "cuda_graph")):
        """Free device memory by tag (``weights`` / ``kv_cache`` / ``cuda_graph``)
        while the trainer uses the GPU (relax/distributed/ray/rollout.py:1201-1233)."""
        if self.running or self.waiting:
            raise RuntimeError("cannot release memory with requests in flight; abort or drain first")
        if "cuda_graph" in tags and not self.memory_saver:
            # without stable addresses the graphs point at freed memory: drop them (re-captured on demand)
            self._graphs = {}
            self._graph_pool = None
        if "kv_cache" in tags:
            if self.memory_saver:
                self._kv_buf.pause()
            else:
                self.kv = None
        if "weights" in tags:
            self.weights.release()
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    def resume_memory_occupation(self, tags: Sequence[str] = ("kv_cache",)):
        if self.memory_saver and self.device.type == "cuda":
            # pausable buffers take physical memory straight from the driver: hand back what the trainer's
            # caching allocator no longer uses first
            torch.cuda.empty_cache()
        if "weights" in tags:
            self.weights.resume()
        if "kv_cache" in tags and (self.kv is None or (self._kv_buf is not None and self._kv_buf.paused)):
            self._alloc_kv()

    def close(self):
        """Destroy the captured CUDA graphs (and their device buffers).  Must run before the process groups are
        destroyed: under tensor parallelism the graphs contain NCCL collectives (embedding all-reduce, logits
        all-gather), and NCCL keeps a communicator alive - its destroy call polls forever - while a graph that
        captured its operations exists."""
        import gc

        if self.device.type == "cuda":
            torch.cuda.synchronize()
        for st in self._graphs.values():
            st.pop("graph", None)
            st.pop("run", None)
        self._graphs = {}
        self._graph_pool = None
        gc.collect()
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    def flush_cache(self):
        if self.running:
            raise RuntimeError("flush_cache with running requests")
        self.bm = BlockManager(self.bm.num_blocks, self.block_size)
        if self.use_cuda_graph or self.windowed_decode:
            self._scratch_block = self.bm.alloc()
        for st in self._graphs.values():     # device-resident batch state refers to blocks of the old manager
            st["rows"] = None

    # ------------------------------------------------------------------ requests
    def attach_vision(self, encoder):
        """Give the engine the vision tower that turns a request's image patches into embeddings at prefill
        (SGLang loads the tower inside the engine: relax/backends/sglang/sglang_engine.py; here the colocated runner
        hands over the trainer's module, a disaggregated engine builds its own and receives its weights by sync)."""
        self.vision = encoder

    def add_request(self, prompt: Sequence[int], params: SamplingParams, group_key: Optional[int] = None,
                    resume_output: Optional[Sequence[int]] = None, resume_logprobs: Optional[Sequence[float]] = None,
                    pixel_patches: Optional[torch.Tensor] = None, grid_thw=None,
                    image_embeds: Optional[torch.Tensor] = None) -> int:
        """Queue a prompt.  With images: ``prompt`` holds one run of ``cfg.image_token_id`` placeholders per image
        (``t * h/merge * w/merge`` tokens), ``grid_thw`` the patch grid of every image, and either the patches
        (an attached vision tower embeds them at prefill) or ready ``image_embeds``.  Requests that share a
        ``group_key`` must carry the same prompt AND the same images: followers reuse the leader's prompt KV."""
        r = Request(self._next_rid, list(prompt), params, group_key, t_arrive=time.perf_counter())
        if grid_thw is not None:
            from ..models.vision import mrope_positions

            if self.cfg.image_token_id < 0 or self.cfg.mrope_section is None:
                raise ValueError(f"model {self.cfg.name} takes no images (no image token / M-RoPE sections)")
            if pixel_patches is None and image_embeds is None:
                raise ValueError("grid_thw given without pixel_patches or image_embeds")
            if pixel_patches is not None and image_embeds is None and getattr(self, "vision", None) is None:
                raise ValueError("pixel_patches need a vision tower: call attach_vision() or pass image_embeds")
            grid = torch.as_tensor(grid_thw, dtype=torch.long).reshape(-1, 3)
            merge = self.cfg.vision.spatial_merge_size if self.cfg.vision is not None else 2
            mp = mrope_positions(r.prompt, grid.tolist(), self.cfg.image_token_id, merge)
            r.mrope_positions = mp.tolist()
            r.pos_delta = int(mp.max()) + 1 - len(r.prompt)
            r.pixel_patches, r.grid_thw, r.image_embeds = pixel_patches, grid, image_embeds
        if resume_output:
            # partial rollout: earlier tokens become part of the context, generation continues
            r.output = list(resume_output)
            r.logprobs = list(resume_logprobs or [0.0] * len(r.output))
        self._next_rid += 1
        self.waiting.append(r)
        return r.rid

    def pause_generation(self):
        self.paused = True

    def continue_generation(self):
        self.paused = False

    def abort_all(self) -> list[Request]:
        """Stop every request; running ones are returned with their partial output."""
        out = []
        for r in self.running:
            self.bm.release(r.blocks)
            r.blocks = []
            r.status, r.finish_reason = "aborted", "abort"
            out.append(r)
        for r in self.waiting:
            r.status, r.finish_reason = "aborted", "abort"
            out.append(r)
        self.running, self.waiting = [], deque()
        return out

    @property
    def has_work(self) -> bool:
        return bool(self.running or self.waiting)

    # ------------------------------------------------------------------ scheduling
    def _admit(self) -> list[Request]:
        """Move waiting requests to running while KV blocks (reserved for their
        whole maximum length) and the prefill token budget allow."""
        admitted, budget = [], self.max_prefill_tokens
        leaders: dict = {}
        while self.waiting and len(self.running) + len(admitted) < self.max_running:
            r = self.waiting[0]
            ctx = r.num_tokens
            need_total = self.bm.blocks_for(len(r.prompt) + r.params.max_new_tokens)
            lead = leaders.get(r.group_key) if (r.group_key is not None and not r.output) else None
            shared_full = (len(r.prompt) - 1) // self.block_size if lead is not None else 0
            need = need_total - shared_full
            reserved = sum(getattr(x, "_reserve", 0) for x in self.running) + sum(getattr(x, "_reserve", 0) for x in admitted)
            if need > self.bm.num_free - reserved:
                break
            if lead is None and ctx > budget and admitted:
                break
            self.waiting.popleft()
            r._lead = lead
            if lead is None:
                budget -= ctx
                if r.group_key is not None and not r.output:
                    leaders[r.group_key] = r
                nb = self.bm.blocks_for(ctx)
                r.blocks = [self.bm.alloc() for _ in range(nb)]
            else:
                # share the leader's full prompt blocks; own the tail block (copied after prefill)
                r.blocks = [self.bm.share(b) for b in lead.blocks[:shared_full]]
                r.blocks += [self.bm.alloc() for _ in range(self.bm.blocks_for(ctx) - shared_full)]
                r.cached_tokens = shared_full * self.block_size
            r._reserve = need_total - len(r.blocks)
            r.status = "running"
            admitted.append(r)
        return admitted

    def _slots(self, r: Request, start: int, end: int) -> list:
        bs = self.block_size
        return [r.blocks[p // bs] * bs + p % bs for p in range(start, end)]

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self) -> list[Request]:
        """One scheduler iteration: admit + prefill new requests, else one decode
        step for all running requests.  Returns requests that finished."""
        if self.paused:
            return []
        self.stats["steps"] += 1
        new = self._admit()
        if new:
            self._prefill(new)
            self.running.extend(new)
        elif self.running:
            self._decode()
        done = [r for r in self.running if r.status == "finished"]
        if done:
            self.running = [r for r in self.running if r.status != "finished"]
            for r in done:
                self.bm.release(r.blocks)
                r.blocks = []
                r._reserve = 0
                r.t_done = time.perf_counter()
        return done

    def _stage(self, arrays):
        """Host lists -> device tensors through a pinned staging buffer and ONE asynchronous host-to-device
        copy.  ``arrays`` is a list of ``(list, dtype)``.  Pinned and device buffers come in pairs that alternate;
        a pinned buffer is rewritten only after the copy that last read it has completed (its event)."""
        if self.device.type != "cuda":
            return [torch.tensor(a, dtype=dt) for a, dt in arrays]
        cpu = [torch.tensor(a, dtype=dt) for a, dt in arrays]
        offs, n = [], 0
        for t in cpu:
            offs.append(n)
            n += (t.numel() * t.element_size() + 15) // 16 * 16
        if getattr(self, "_pin", None) is None or self._pin[0].numel() < n:
            if getattr(self, "_pin_ev", None) is not None:
                for ev in self._pin_ev:
                    ev.synchronize()
            cap = max(n * 2, 1 << 16)
            self._pin = [torch.empty(cap, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
            self._dev_stage = [torch.empty(cap, dtype=torch.uint8, device=self.device) for _ in range(2)]
            self._pin_ev = [torch.cuda.Event() for _ in range(2)]
            for ev in self._pin_ev:
                ev.record()
            self._stage_flip = 0
        self._stage_flip ^= 1
        pin, dbuf, ev = self._pin[self._stage_flip], self._dev_stage[self._stage_flip], self._pin_ev[self._stage_flip]
        ev.synchronize()
        for t, o in zip(cpu, offs):
            nb = t.numel() * t.element_size()
            if nb:
                pin[o:o + nb].copy_(t.view(-1).view(torch.uint8))
        if n:
            dbuf[:n].copy_(pin[:n], non_blocking=True)
            ev.record()
        self.stats["h2d_bytes"] = self.stats.get("h2d_bytes", 0) + n
        out = []
        for t, o in zip(cpu, offs):
            nb = t.numel() * t.element_size()
            out.append(dbuf[o:o + nb].view(t.dtype).view(t.shape))
        return out

    def _prefill(self, reqs: list[Request]):
        leaders = [r for r in reqs if r._lead is None]
        toks, pos, cu, slots, last_rows = [], [], [0], [], []
        multimodal = any(r.mrope_positions is not None for r in leaders)
        pos3 = [[], [], []]
        for r in leaders:
            ctx = r.prompt + r.output
            toks += ctx
            if multimodal:       # M-RoPE ids: three streams (equal for text), generated tokens continue after the prompt's maximum
                mp = r.mrope_positions or [list(range(len(r.prompt)))] * 3
                tail = [len(r.prompt) + r.pos_delta + i for i in range(len(r.output))]
                for a in range(3):
                    pos3[a] += list(mp[a]) + tail
            else:
                pos += list(range(len(ctx)))
            slots += self._slots(r, 0, len(ctx))
            cu.append(cu[-1] + len(ctx))
            last_rows.append(cu[-1] - 1)
        dev = self.device
        if leaders:
            t, pos_t, cu_t, slots_t, last_t = self._stage([(toks, torch.int64), (pos3 if multimodal else pos, torch.int64),
                                                           (cu, torch.int32), (slots, torch.int64), (last_rows, torch.int64)])
            image = self._image_rows(leaders, cu, toks) if multimodal else None
            if self.return_routed_experts:
                self.weights.routing_capture = []
            h_all = None
            if self.hybrid:
                self.weights.seq_ctx = {"mode": "prefill", "cu": list(cu), "cu_t": cu_t, "out": {}, "positions": pos_t,
                                        "cap": [len(r.prompt) + r.params.max_new_tokens for r in leaders]}
            if self.speculative:
                logits, h_all = self.weights.forward_prefill(t, pos_t, cu_t, slots_t, self.kv, last_t, self.tp,
                                                             max_seqlen=max(b - a for a, b in zip(cu, cu[1:])), return_hidden=True)
            else:
                logits = self.weights.forward_prefill(t, pos_t, cu_t, slots_t, self.kv, last_t, self.tp,
                                                      max_seqlen=max(b - a for a, b in zip(cu, cu[1:])), image=image)
            self.stats["prefill_tokens"] += len(toks)
            if self.hybrid:
                out = self.weights.seq_ctx["out"]
                for j, r in enumerate(leaders):
                    st = {i: out[i][j] for i in out}
                    r._gdn, r._mla = ({}, st) if self.latent else (st, {})
                self.weights.seq_ctx = None
            if self.return_routed_experts:
                routed = torch.stack(self.weights.routing_capture, 1).tolist()      # [T][L_moe][k]
                self.weights.routing_capture = None
                for r, a, b in zip(leaders, cu, cu[1:]):
                    r.routed_experts = routed[a:b]
        row_of = {id(r): i for i, r in enumerate(leaders)}
        # followers copy the leader's partially filled tail block and reuse its last-token logits
        rows = []
        bs = self.block_size
        for r in reqs:
            lead = r._lead
            if lead is not None:
                n_shared = (len(r.prompt) - 1) // bs
                for j in range(n_shared, len(lead.blocks)):
                    if j < len(r.blocks):
                        self.kv[:, :, r.blocks[j]] = self.kv[:, :, lead.blocks[j]]
                self.stats["cached_tokens"] += len(r.prompt)
                if self.hybrid:          # the same prompt leaves the same recurrent state / the same latent rows
                    r._gdn = {i: [c.clone(), S.clone()] for i, (c, S) in lead._gdn.items()}
                    r._mla = {i: [a.clone(), None if b is None else b.clone()] for i, (a, b) in lead._mla.items()}
                rows.append(row_of[id(lead)])
                if self.return_routed_experts:
                    r.routed_experts = [list(x) for x in lead.routed_experts[:len(r.prompt)]]
            else:
                rows.append(row_of[id(r)])
        sel = logits[torch.tensor(rows, device=dev)] if rows != list(range(len(leaders))) else logits
        self._sample_and_append(reqs, sel)
        if self.speculative and leaders:
            self._draft_after_prefill(reqs, leaders, h_all, cu, slots_t, pos_t, cu_t, row_of)
        now = time.perf_counter()
        for r in reqs:
            r.t_first = now

    def _image_rows(self, leaders, cu, toks):
        """``(rows, embeds)``: the packed rows of this prefill that are image placeholders and what goes there.
        All images of the batch pass through the vision tower in one call."""
        img_id = self.cfg.image_token_id
        rows, ready, patches, grids = [], [], [], []
        for r, a in zip(leaders, cu):
            if r.grid_thw is None:
                continue
            rows += [a + i for i, tk in enumerate(r.prompt) if tk == img_id]
            if r.image_embeds is not None:
                ready.append(("e", r.image_embeds))
            else:
                ready.append(("p", len(patches)))
                patches.append(r.pixel_patches)
                grids.append(r.grid_thw)
        if not rows:
            return None
        embeds_of_patches = None
        if patches:
            tower = self.vision
            wdev = tower.patch_embed.device
            out = tower(torch.cat([p.to(wdev) for p in patches]), torch.cat(grids).to(wdev))
            m2 = tower.cfg.spatial_merge_size ** 2
            counts = [int((g[:, 0] * g[:, 1] * g[:, 2]).sum()) // m2 for g in grids]
            embeds_of_patches = list(out.split(counts))
        parts = [(e if kind == "e" else embeds_of_patches[e]).to(self.device) for kind, e in ready]
        emb = torch.cat(parts)
        if emb.shape[0] != len(rows):
            raise ValueError(f"{len(rows)} image placeholder tokens in the batch but {emb.shape[0]} image embeddings")
        return torch.tensor(rows, dtype=torch.int64, device=self.device), emb

    def _decode(self):
        if self.speculative:
            return self._decode_speculative()
        if self.windowed_decode and self._decode_window():
            return
        reqs = self.running
        dev = self.device
        bs = self.block_size
        # the newest token of each request is fed; its K/V goes to position num_tokens-1
        for r in reqs:
            p = r.num_tokens - 1
            if p // bs >= len(r.blocks):
                r.blocks.append(self.bm.alloc())
                r._reserve = max(0, r._reserve - 1)
        B = len(reqs)
        maxb = max(len(r.blocks) for r in reqs)
        maxb = (maxb + 7) // 8 * 8
        bt_rows = [r.blocks + [0] * (maxb - len(r.blocks)) for r in reqs]
        tok, pos, ctx, slots, bt = self._stage([
            ([(r.output[-1] if r.output else r.prompt[-1]) for r in reqs], torch.int64),
            ([r.num_tokens - 1 + r.pos_delta for r in reqs], torch.int64),
            ([r.num_tokens for r in reqs], torch.int32),
            ([r.blocks[(r.num_tokens - 1) // bs] * bs + (r.num_tokens - 1) % bs for r in reqs], torch.int64),
            (bt_rows, torch.int32)])
        if self.return_routed_experts:
            self.weights.routing_capture = []
        if self.hybrid:
            layers = list(reqs[0]._gdn)
            self.weights.seq_ctx = {"mode": "decode", "positions": pos,
                                    "state": {i: [torch.stack([r._gdn[i][0] for r in reqs]),
                                                  torch.stack([r._gdn[i][1] for r in reqs])] for i in layers},
                                    "cache": {i: [r._mla[i] for r in reqs] for i in reqs[0]._mla},
                                    "lens": [r.num_tokens - 1 for r in reqs]}
        logits = self.weights.forward_decode(tok, pos, bt, ctx, slots, self.kv, self.tp)
        if self.hybrid:
            st = self.weights.seq_ctx["state"]
            for j, r in enumerate(reqs):
                r._gdn = {i: [st[i][0][j], st[i][1][j]] for i in st}
            self.weights.seq_ctx = None
        if self.return_routed_experts:
            routed = torch.stack(self.weights.routing_capture, 1).tolist()
            self.weights.routing_capture = None
            for r, x in zip(reqs, routed):
                r.routed_experts.append(x)
        self.stats["decode_tokens"] += B
        self._sample_and_append(reqs, logits)

    # ------------------------------------------------------------------ windowed decode (CUDA graph of one step)
    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)
    N_STOP = 4      # stop ids per row known to the device; longer lists are still honoured by the host

    def _window_state(self, bucket: int):
        """Device-resident batch state, window ring and (on CUDA) the captured graph of one decode step for one
        batch-size bucket.  Two regions of ONE pinned host mirror: the per-window part (step counter, uniform draws)
        is uploaded before every window, the batch part (tokens, positions, block tables, sampling parameters, stop
        rules) only when the set of running requests changed."""
        st = self._graphs.get(bucket)
        if st is not None:
            return st
        dev, bs = self.device, self.block_size
        maxb = (self.bm.blocks_for(self._max_model_len()) + 7) // 8 * 8
        W = self.decode_window
        i64, i32, f32 = torch.int64, torch.int32, torch.float32
        per_window = [("counter", i32, (4,)), ("u", f32, (bucket,)), ("u_all", f32, (W, bucket))]
        per_batch = [("tok", i64, (bucket,)), ("pos", i64, (bucket,)), ("slots", i64, (bucket,)), ("topk", i64, (bucket,)),
                     ("eos", i64, (bucket,)), ("stop", i64, (bucket, self.N_STOP)), ("ctx", i32, (bucket,)),
                     ("active", i32, (bucket,)), ("remain", i32, (bucket,)), ("bt", i32, (bucket, maxb)),
                     ("temp", f32, (bucket,)), ("topp", f32, (bucket,)), ("delta", i64, (bucket,))]
        offs, n = {}, 0
        for name, dt, shp in per_window + per_batch:
            if name == "tok":
                n_window = n
            offs[name] = n
            n += (math.prod(shp) * torch.empty(0, dtype=dt).element_size() + 15) // 16 * 16
        cuda = dev.type == "cuda"
        host = torch.zeros(n, dtype=torch.uint8, pin_memory=cuda)
        devb = torch.zeros(n, dtype=torch.uint8, device=dev)

        def views(buf):
            out = {}
            for name, dt, shp in per_window + per_batch:
                nb = math.prod(shp) * torch.empty(0, dtype=dt).element_size()
                out[name] = buf[offs[name]:offs[name] + nb].view(dt).view(shp)
            return out

        st = {"host": host, "dev": devb, "h": views(host), "d": views(devb), "nbytes": n, "n_window": n_window,
              "maxb": maxb, "rows": None, "bucket": bucket}
        d = st["d"]
        d["out_tok"] = torch.full((W, bucket), -1, dtype=i64, device=dev)
        d["out_lp"] = torch.zeros(W, bucket, dtype=f32, device=dev)
        st["host_tok"] = torch.zeros(W, bucket, dtype=i64, pin_memory=cuda)
        st["host_lp"] = torch.zeros(W, bucket, dtype=f32, pin_memory=cuda)
        self._pad_rows(st, 0, bucket)
        devb.copy_(host)
        counter = d["counter"]
        d["counter"] = counter[:1]

        if self.return_routed_experts:
            nl, k = len(self.weights.moe_layers), self.cfg.moe_top_k
            d["out_routed"] = torch.zeros(W, bucket, nl, k, dtype=torch.int32, device=dev)
            st["host_routed"] = torch.zeros(W, bucket, nl, k, dtype=torch.int32, pin_memory=cuda)

        def run():
            if self.return_routed_experts:
                self.weights.routing_capture = []
            # rotary position = cache position + the row's offset (non-zero after an image: M-RoPE advances by the
            # largest grid side, not by the number of placeholder tokens)
            rope_pos = d["pos"] + d["delta"] if self.cfg.mrope_section is not None else d["pos"]
            logits = self.weights.forward_decode(d["tok"], rope_pos, d["bt"], d["ctx"], d["slots"], self.kv, self.tp)
            if self.return_routed_experts:      # ring slot = the step counter, read on the device (before it advances)
                routed = torch.stack(self.weights.routing_capture, 1).to(torch.int32)
                self.weights.routing_capture = None
                d["out_routed"].index_copy_(0, d["counter"].long().clamp_max(W - 1), routed.unsqueeze(0))
            tok, lp = ops.sample(logits[:, :self.cfg.vocab_size], d["temp"], d["topk"], d["topp"], d["u"])
            ops.decode_advance(tok, lp, d, bs)

        st["run"] = run
        if self.use_cuda_graph:
            run()                                   # eager warm-up (lazy initialisation, communicator set-up)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=self._graph_pool):
                run()
            if self._graph_pool is None:
                self._graph_pool = g.pool()
            st["graph"] = g
            devb.copy_(host)                        # the warm-up and the capture advanced the padding rows' ring index
        self._graphs[bucket] = st
        return st

    def _pad_rows(self, st, lo: int, hi: int):
        """Neutral padding rows: a stopped row with a context of one token held in the scratch block."""
        h, bs = st["h"], self.block_size
        h["tok"][lo:hi] = 0
        h["pos"][lo:hi] = 0
        h["delta"][lo:hi] = 0
        h["ctx"][lo:hi] = 1
        h["bt"][lo:hi] = self._scratch_block
        h["slots"][lo:hi] = self._scratch_block * bs
        h["temp"][lo:hi] = 1.0
        h["topp"][lo:hi] = 1.0
        h["topk"][lo:hi] = -1
        h["eos"][lo:hi] = -1
        h["stop"][lo:hi] = -1
        h["active"][lo:hi] = 0
        h["remain"][lo:hi] = 0

    def _max_model_len(self) -> int:
        return getattr(self, "max_model_len", 0) or 4096

    def _decode_window(self) -> bool:
        """Up to ``decode_window`` decode steps for the running batch with one host round trip.  Returns False when
        the batch does not fit a bucket or the model length (the caller then takes the host-driven step)."""
        reqs = self.running
        bs = self.block_size
        B = len(reqs)
        bucket = next((b for b in self.GRAPH_BUCKETS if b >= B), None)
        if bucket is None or any(len(r.prompt) + r.params.max_new_tokens > self._max_model_len() for r in reqs):
            return False
        # the device advances positions on its own: hand every request all the blocks it can ever need now (they
        # were already counted against the free pool at admission)
        for r in reqs:
            need = self.bm.blocks_for(len(r.prompt) + r.params.max_new_tokens)
            while len(r.blocks) < need:
                r.blocks.append(self.bm.alloc())
            r._reserve = 0
        st = self._window_state(bucket)
        h, d = st["h"], st["d"]
        W = min(self.decode_window, max(r.params.max_new_tokens - len(r.output) for r in reqs))
        rows = tuple(r.rid for r in reqs)
        fresh = st["rows"] != rows
        if fresh:
            maxb = st["maxb"]
            last = [(r.output[-1] if r.output else r.prompt[-1]) for r in reqs]
            npos = [r.num_tokens - 1 for r in reqs]
            h["tok"][:B] = torch.tensor(last, dtype=torch.int64)
            h["pos"][:B] = torch.tensor(npos, dtype=torch.int64)
            h["ctx"][:B] = torch.tensor([p + 1 for p in npos], dtype=torch.int32)
            h["delta"][:B] = torch.tensor([r.pos_delta for r in reqs], dtype=torch.int64)
            h["slots"][:B] = torch.tensor([r.blocks[p // bs] * bs + p % bs for r, p in zip(reqs, npos)], dtype=torch.int64)
            h["bt"][:B] = torch.tensor([r.blocks + [self._scratch_block] * (maxb - len(r.blocks)) for r in reqs], dtype=torch.int32)
            h["temp"][:B] = torch.tensor([r.params.temperature for r in reqs], dtype=torch.float32)
            h["topk"][:B] = torch.tensor([r.params.top_k for r in reqs], dtype=torch.int64)
            h["topp"][:B] = torch.tensor([r.params.top_p for r in reqs], dtype=torch.float32)
            h["eos"][:B] = torch.tensor([(-1 if (r.params.ignore_eos or self.eos is None) else self.eos) for r in reqs], dtype=torch.int64)
            stops = [([-1] if r.params.ignore_eos else list(r.params.stop_token_ids)[:self.N_STOP]) for r in reqs]
            h["stop"][:B] = torch.tensor([s_ + [-1] * (self.N_STOP - len(s_)) for s_ in stops], dtype=torch.int64)
            h["active"][:B] = 1
            h["remain"][:B] = torch.tensor([r.params.max_new_tokens - len(r.output) for r in reqs], dtype=torch.int32)
            if B < bucket:
                self._pad_rows(st, B, bucket)
            st["rows"] = rows
        h["counter"][:] = 0
        for i in range(W):      # one draw per step, in the order the host-driven loop makes them
            h["u_all"][i, :B] = torch.rand(B, generator=self.gen)
        h["u"][:] = h["u_all"][0]
        nb = st["nbytes"] if fresh else st["n_window"]
        st["dev"][:nb].copy_(st["host"][:nb], non_blocking=True)
        if "graph" in st:
            for _ in range(W):
                st["graph"].replay()
        else:
            for _ in range(W):
                st["run"]()
        st["host_tok"][:W].copy_(d["out_tok"][:W], non_blocking=True)
        st["host_lp"][:W].copy_(d["out_lp"][:W], non_blocking=True)
        if self.return_routed_experts:
            st["host_routed"][:W].copy_(d["out_routed"][:W], non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()    # also completes the upload: the mirror may be rewritten
        tok_w, lp_w = st["host_tok"][:W, :B].tolist(), st["host_lp"][:W, :B].tolist()
        self.stats["h2d_bytes"] = self.stats.get("h2d_bytes", 0) + nb
        self.stats["d2h_bytes"] = self.stats.get("d2h_bytes", 0) + W * bucket * 12
        self.stats["graph_replays"] = self.stats.get("graph_replays", 0) + W
        self.stats["steps"] += W - 1
        routed_w = st["host_routed"][:W, :B].tolist() if self.return_routed_experts else None
        for i in range(W):
            live = [(j, r) for j, r in enumerate(reqs) if r.status == "running"]
            if not live:
                break
            if routed_w is not None:
                for j, r in live:
                    r.routed_experts.append(routed_w[i][j])
            row_t, row_l = tok_w[i], lp_w[i]
            if any(row_t[j] < 0 for j, _ in live):
                raise RuntimeError("decode window: the device stopped a row the host still considers running")
            self.stats["decode_tokens"] += len(live)
            self._append_tokens([r for _, r in live], [row_t[j] for j, _ in live], [row_l[j] for j, _ in live])
        if any(r.status != "running" for r in reqs):
            st["rows"] = None
        return True

    def _sample_and_append(self, reqs: list[Request], logits: torch.Tensor):
        dev = self.device
        B = len(reqs)
        v = self.cfg.vocab_size
        logits = logits[:, :v]
        u = torch.rand(B, generator=self.gen)
        temp, topk, topp, u = self._stage([([r.params.temperature for r in reqs], torch.float32),
                                           ([r.params.top_k for r in reqs], torch.int64),
                                           ([r.params.top_p for r in reqs], torch.float32),
                                           (u.tolist(), torch.float32)])
        tok, lp = ops.sample(logits, temp, topk, topp, u)
        tok_l, lp_l = tok.tolist(), lp.tolist()
        self.stats["d2h_bytes"] = self.stats.get("d2h_bytes", 0) + B * 12
        self._append_tokens(reqs, tok_l, lp_l)

    def _append_tokens(self, reqs, tok_l, lp_l):
        for r, t, l in zip(reqs, tok_l, lp_l):
            r.output.append(t)
            r.logprobs.append(l)
            r.weight_versions.append(self.weight_version)
            stop = (not r.params.ignore_eos) and ((self.eos is not None and t == self.eos) or t in r.params.stop_token_ids)
            if stop:
                r.status, r.finish_reason = "finished", "stop"
            elif len(r.output) >= r.params.max_new_tokens:
                r.status, r.finish_reason = "finished", "length"

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams],
                 group_keys: Optional[Sequence[int]] = None, images: Optional[Sequence[Optional[dict]]] = None) -> list[Request]:
        """Blocking generation of a batch; results in the order of ``prompts``.  ``images[i]`` is None or a dict with
        ``grid_thw`` and ``pixel_patches`` (or ``image_embeds``) of prompt ``i``."""
        ids = []
        for i, p in enumerate(prompts):
            sp = params if isinstance(params, SamplingParams) else params[i]
            im = images[i] if images is not None else None
            ids.append(self.add_request(p, sp, group_keys[i] if group_keys is not None else None,
                                        **({k: im.get(k) for k in ("pixel_patches", "grid_thw", "image_embeds")} if im else {})))
        res = {}
        while self.has_work:
            for r in self.step():
                res[r.rid] = r
        return [res[i] for i in ids]

    def update_weight_version(self, v: int):
        self.weight_version = v
