"""Policy trainer rank (``actor`` / ``actor_fwd`` / ``reference`` / ``critic`` roles).

One :class:`TrainActor` lives in each trainer process.  It owns the model
shard, the distributed optimizer and tagged weight snapshots (``actor``,
``ref``, ``old_actor``, ``teacher``), and exposes the operations the reference's
trainer actor offers (relax/backends/megatron/actor.py:177: ``train``,
``compute_log_prob``, ``update_weights``, ``save_model``, ``sleep`` / ``wake_up``).

A training call follows relax/backends/megatron/actor.py:890-1096:
reference log-probs -> old-policy log-probs -> advantages -> optimizer steps.
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist

from ..algo import loss as L
from ..algo.ppo_utils import Segments, post_process_rewards
from ..data.packing import pack_samples
from ..data.seqlen_balancing import balanced_microbatches, karmarkar_karp
from ..models.config import ModelConfig
from ..models.transformer import GPTModel
from ..parallel.state import ParallelState, single_process_state
from ..utils.timer import Timer
from .optimizer import DistributedOptimizer, OptimizerConfig


@dataclass
class TrainConfig:
    advantage_estimator: str = "grpo"
    global_batch_size: int = 32            # samples per optimizer step (all DP ranks together)
    max_tokens_per_gpu: int = 8192         # dynamic micro-batch token cap
    use_dynamic_batch_size: bool = True
    micro_batch_size: int = 1
    rollout_temperature: float = 1.0
    n_samples_per_prompt: int = 8
    kl_coef: float = 0.0                   # reward shaping (ppo / reinforce++)
    gamma: float = 1.0
    lambd: float = 1.0
    normalize_advantages: bool = False
    rewards_normalization: bool = True
    grpo_std_normalization: bool = True
    balance_data: bool = False
    recompute: bool = False
    compute_advantages_and_returns: bool = True   # False (--disable-compute-advantages-and-returns): a custom loss brings its own
    use_rollout_entropy: bool = False         # forward-only actor / reference passes also return per-token entropies
    problem_type: Optional[str] = None        # sequence classification: single_label_classification (default) / multi_label_classification
    classification_threshold: float = 0.5     # multi-label: sigmoid threshold of the accuracy metrics
    pad_multiple: int = 128
    # context parallelism: every zig-zag chunk is padded to a multiple of this many tokens (None: ``pad_multiple``
    # on a GPU, where the attention tiles want whole 128-row blocks, 1 on the CPU)
    cp_chunk_multiple: Optional[int] = None
    # context-parallel attention: "peer" (GPU default: K/V staged once in every peer's memory over NVLink, partial
    # results merged by log-sum-exp), "allgather" (K/V gathered, two plain attention calls per rank; --allgather-cp),
    # "ring" (send/recv ring with the PyTorch statement of attention: the CPU oracle)
    cp_attention: Optional[str] = None
    use_rollout_logprobs: bool = False
    keep_old_actor: bool = False
    compute_entropy: bool = True
    ref_on_host: bool = False           # keep the frozen reference weights in pinned host memory
    lora: Optional[object] = None       # a train.lora.LoRAConfig: train adapters only
    # regular expressions on parameter names: freeze the matches / train only the matches
    # (relax/backends/megatron/model_provider.py freeze :603-639)
    freeze_params_name_list: Optional[Sequence[str]] = None
    only_train_params_name_list: Optional[Sequence[str]] = None
    # MoE: the expert choices of the old-policy forward are replayed in the training forward, so both evaluate the
    # same experts (--use-routing-replay; relax/backends/megatron/actor.py fill_routing_replay :534-641)
    use_routing_replay: bool = False
    # R3: replay the expert choices the ROLLOUT engine made (batch field ``rollout_routed_experts``) in the old-policy
    # and training forwards (relax/backends/sglang/routing_replay_patch.py, --use-rollout-routing-replay)
    use_rollout_routing_replay: bool = False
    # on-policy distillation: per-token divergence between the policy and a teacher on the sampled tokens, applied to
    # the advantages as a dense penalty (relax/utils/opd/opd_utils.py apply_opd_to_advantages :1275).  The teacher's
    # log-probs come with the batch (``teacher_log_probs``, external teacher) or from the ``teacher`` weight snapshot.
    opd_kl_coef: float = 0.0
    opd_kl_type: str = "reverse_kl"
    opd_token_selection: str = "sampled_token"     # or student_topk / teacher_topk / union (with opd_log_prob_top_k)
    opd_log_prob_top_k: int = 0
    opd_jsd_alpha: float = 0.5
    opd_norm_mode: str = "tail"
    opd_log_prob_min_clamp: Optional[float] = None
    opd_only_reward: bool = False                  # drop the task reward's advantages, keep the distillation signal
    opd_per_token_clip: Optional[float] = None
    enable_mtp_training: bool = False   # add the multi-token-prediction loss of the model's MTP blocks
    mtp_loss_scaling_factor: float = 0.1
    mtp_only_training: bool = False     # freeze the trunk, train the MTP blocks alone
    ci: Optional[object] = None         # a train.ci_utils.CIConfig: first-step KL checks, grad-norm record / compare
    loss: L.LossConfig = field(default_factory=L.LossConfig)
    optim: OptimizerConfig = field(default_factory=OptimizerConfig)


def _shift_mask(mask: torch.Tensor, response_lengths: Sequence[int], k: int) -> torch.Tensor:
    """``out[j] = mask[j + k]`` inside each sample's response span, 0 past its end."""
    out = torch.zeros_like(mask)
    o = 0
    for R in response_lengths:
        if R > k:
            out[o:o + R - k] = mask[o + k:o + R]
        o += R
    return out


def concat_batches(parts: Sequence[dict]) -> dict:
    """Join row-wise batches (field -> one entry per row); scalar fields must agree and are kept once."""
    out: dict = {}
    for k in parts[0]:
        v0 = parts[0][k]
        if isinstance(v0, list):
            out[k] = [x for p in parts for x in p[k]]
        elif torch.is_tensor(v0) and v0.dim() > 0:
            out[k] = torch.cat([p[k] for p in parts])
        else:
            out[k] = v0
    return out


class TrainActor:
    def __init__(self, model_cfg: ModelConfig, cfg: TrainConfig, ps: Optional[ParallelState] = None,
                 device="cpu", seed: int = 0, role: str = "actor", with_optimizer: bool = True,
                 with_reference: bool = False):
        self.mcfg, self.cfg, self.role = model_cfg, cfg, role
        self.ps = ps or single_process_state()
        self.device = torch.device(device)
        self.model = GPTModel(model_cfg, self.ps, device=device, seed=seed, recompute=cfg.recompute)
        if model_cfg.vision is not None:
            # vision-language model: the tower is a sub-module of the language model, so the optimizer, checkpoints
            # and snapshots see its parameters like any other (relax/backends/megatron/model_provider.py builds the
            # VL model the same way: one module tree)
            from ..models.vision import VisionEncoder, vision_config_from_model

            if self.ps.pp.size > 1 or self.ps.cp.size > 1:
                raise NotImplementedError("vision-language training runs with pp = cp = 1")
            self.model.vision = VisionEncoder(vision_config_from_model(model_cfg), dtype=self.model.dtype, device=device,
                                              seed=seed + 17)
        self.ep_comm = None
        if (self.device.type == "cuda" and self.ps.ep.size > 1 and model_cfg.is_moe
                and os.environ.get("RELAX_B200_EP_PEER", "1") == "1"):
            self._attach_ep_comm()
        if cfg.lora is not None:
            from .lora import apply_lora

            apply_lora(self.model, cfg.lora)
        if cfg.mtp_only_training:
            for n, p in self.model.named_parameters():
                p.requires_grad_(n.startswith("mtp."))
        if cfg.freeze_params_name_list or cfg.only_train_params_name_list:
            import re

            fr = [re.compile(x) for x in (cfg.freeze_params_name_list or [])]
            only = [re.compile(x) for x in (cfg.only_train_params_name_list or [])]
            for n, p in self.model.named_parameters():
                if not p.requires_grad:
                    continue
                if any(r.search(n) for r in fr) or (only and not any(r.search(n) for r in only)):
                    p.requires_grad_(False)
            if not any(p.requires_grad for p in self.model.parameters()):
                raise ValueError("the freeze lists leave no trainable parameter")
        self.optimizer = DistributedOptimizer(self.model, self.ps, cfg.optim) if with_optimizer else None
        self.timer = Timer()
        # trajectory replay capture (utils/replay.py): off unless RELAX_REPLAY_CAPTURE_DIR is set
        from ..utils.replay import ReplayRecorder, run_identity

        self.replay = ReplayRecorder.from_env(
            dist.get_rank() if dist.is_initialized() else 0,
            run_identity(model_cfg.name, cfg.loss, {"dp": [ps.dp.rank, ps.dp.size], "tp": [ps.tp.rank, ps.tp.size],
                                                     "cp": [ps.cp.rank, ps.cp.size], "pp": [ps.pp.rank, ps.pp.size]}, model_cfg.dtype)
        ) if os.environ.get("RELAX_REPLAY_CAPTURE_DIR") else ReplayRecorder(None)
        self._cur_rollout, self._cur_step = -1, 0
        self.weight_version = 0
        self.snapshots: dict[str, torch.Tensor] = {}
        self._active_tag = "actor"
        if self.optimizer is None:
            self._flatten_params()
        if with_reference:
            self.backup("ref", to_host=cfg.ref_on_host)
            if cfg.ref_on_host and self.device.type == "cuda":
                torch.cuda.synchronize()

    def _attach_ep_comm(self):
        """Expert-parallel dispatch / combine by peer stores over NVLink (parallel/ep_peer.py) when the whole EP group
        sits on this node; otherwise the layers keep the NCCL all-to-all.  One communicator serves every MoE layer."""
        import socket

        from ..models.moe import MoEMLP
        from ..parallel.ep_peer import EPComm

        g = self.ps.ep
        hosts = [None] * g.size
        dist.all_gather_object(hosts, socket.gethostname(), group=g.group)
        if len(set(hosts)) != 1:
            return
        rows = self.cfg.max_tokens_per_gpu * self.mcfg.moe_top_k * 2      # room for an uneven routing
        self.ep_comm = EPComm(g, self.device, rows, self.mcfg.hidden_size, max_experts=max(512, self.mcfg.num_experts))
        for mod in self.model.modules():
            if isinstance(mod, MoEMLP):
                mod.ep_comm = self.ep_comm

    # ------------------------------------------------------------------ tagged weights
    def _flatten_params(self):
        ps_ = [p for p in self.model.parameters()]
        n = sum((p.numel() + 15) // 16 * 16 for p in ps_)
        buf = torch.zeros(n, dtype=ps_[0].dtype, device=ps_[0].device)
        o = 0
        self._flat_offsets = []
        for p in ps_:
            v = buf[o:o + p.numel()].view_as(p)
            v.copy_(p.data)
            p.data = v
            self._flat_offsets.append(o)
            o += (p.numel() + 15) // 16 * 16
        self._flat = buf

    @property
    def param_buf(self) -> torch.Tensor:
        return self.optimizer.param_buf if self.optimizer is not None else self._flat

    def _bound_params(self):
        if self.optimizer is not None:
            return list(zip(self.optimizer.params, self.optimizer.offsets))
        return list(zip(self.model.parameters(), self._flat_offsets))

    def backup(self, tag: str, to_host: bool = False):
        """Snapshot the active weights under ``tag`` (device copy, or pinned host
        copy like relax/utils/training/tensor_backper.py:48-80)."""
        src = self.param_buf
        if to_host:
            dst = self.snapshots.get(tag)
            if dst is None or dst.is_cuda or dst.shape != src.shape:
                dst = torch.empty(src.shape, dtype=src.dtype, pin_memory=src.is_cuda)
            dst.copy_(src, non_blocking=True)
        else:
            dst = src.clone()
        self.snapshots[tag] = dst

    def switch_model(self, tag: str):
        """Make the weights stored under ``tag`` the ones the model computes
        with.  Device snapshots are bound by re-pointing the parameter views (no
        copy); host snapshots are copied into a staging buffer first."""
        if tag == self._active_tag:
            return
        if tag == "actor":
            buf = self.param_buf
            self._stage = None      # staging copy of a host snapshot is only needed while it is bound
        else:
            buf = self.snapshots[tag]
            if not buf.is_cuda and self.device.type == "cuda":
                stage = getattr(self, "_stage", None)
                if stage is None:
                    stage = self._stage = torch.empty_like(self.param_buf)
                stage.copy_(buf, non_blocking=True)
                buf = stage
        for p, o in self._bound_params():
            p.data = buf[o:o + p.numel()].view_as(p)
        self._active_tag = tag

    # ------------------------------------------------------------------ forward
    def _pack(self, tokens: Sequence, response_lengths: Sequence[int]):
        mult = self.ps.tp.size * (self.cfg.pad_multiple if self.device.type == "cuda" else 1)
        return pack_samples(tokens, response_lengths, pad_multiple=max(1, mult), device=self.device)

    def _pack_batch(self, batch: dict, ids: Sequence[int]):
        """Pack samples ``ids`` of ``batch``.  With ``multimodal_train_inputs`` (per sample None or a dict with
        ``pixel_patches [N, patch_dim]`` and ``grid_thw [n_img, 3]``; relax/backends/megatron/data.py get_batch
        carries the same field) the packed batch gets M-RoPE positions ``[3, T]`` and the concatenated patches."""
        pb = self._pack([batch["tokens"][i] for i in ids], [batch["response_lengths"][i] for i in ids])
        mm = batch.get("multimodal_train_inputs")
        if self.mcfg.vision is None or mm is None:
            return pb
        from ..models.vision import mrope_positions

        merge = self.mcfg.vision.spatial_merge_size
        pos, patches, grids, img_rows, row0 = [], [], [], [], 0
        for i in ids:
            toks = [int(t) for t in batch["tokens"][i]]
            n_prompt = len(toks) - int(batch["response_lengths"][i])
            m = mm[i]
            if m is None:
                pos.append(torch.arange(len(toks)).expand(3, -1))
                row0 += len(toks)
                continue
            grid = torch.as_tensor(m["grid_thw"], dtype=torch.long).reshape(-1, 3)
            # ids of the prompt from its image grids; the response continues linearly after the prompt's maximum
            pp = mrope_positions(toks[:n_prompt], grid.tolist(), self.mcfg.image_token_id, merge)
            tail = torch.arange(len(toks) - n_prompt) + (int(pp.max()) + 1 if n_prompt else 0)
            pos.append(torch.cat([pp, tail.expand(3, -1)], 1))
            patches.append(torch.as_tensor(m["pixel_patches"]))
            grids.append(grid)
            # placeholders of the PROMPT only: a sampled response token that happens to be the placeholder id is text
            img_rows += [row0 + j for j in range(n_prompt) if toks[j] == self.mcfg.image_token_id]
            row0 += len(toks)
        T = int(pb.tokens.numel())
        used = sum(p.shape[1] for p in pos)
        if used < T:       # the padding sequence
            pos.append(torch.arange(T - used).expand(3, -1))
        pb.positions = torch.cat(pos, 1).to(self.device)
        if patches:
            pb.pixel_patches = torch.cat(patches).to(self.device)
            pb.grid_thw = torch.cat(grids).to(self.device)
            pb.image_rows = torch.tensor(img_rows, dtype=torch.int64, device=self.device)
        return pb

    def _embed_multimodal(self, pb):
        """Token embeddings of a packed batch with the image placeholder rows replaced by the tower's output."""
        if self.ps.tp.size > 1:
            raise NotImplementedError("vision-language training runs with tp = 1 in the trainer")
        emb = self.model.embedding.word_embeddings(pb.tokens, False)
        img = self.model.vision(pb.pixel_patches, pb.grid_thw)
        if img.shape[0] != pb.image_rows.numel():
            raise ValueError(f"{pb.image_rows.numel()} image placeholders in the prompts but {img.shape[0]} image embeddings")
        return emb.index_copy(0, pb.image_rows, img.to(emb.dtype))

    def _forward_logp_cp(self, pb, with_entropy: bool):
        """Context-parallel forward: every sample is sharded zig-zag over the CP ranks (two chunks per rank),
        attention runs as ring attention - or, with a :class:`~relax_b200.parallel.cp_peer.CPComm` attached as
        ``self.cp_comm``, with in-kernel reads of the peers' K/V - and the per-token outputs are gathered so every
        rank evaluates the same loss (gradient flows through the local tokens only)."""
        from ..parallel import cp as CP

        g = self.ps.cp
        cp, r = g.size, g.rank
        mult = self.cfg.cp_chunk_multiple or (self.cfg.pad_multiple if self.device.type == "cuda" else 1)
        unit = 2 * cp * max(1, self.ps.tp.size) * mult
        cu = pb.cu_seqlens.tolist()
        lps, ens = [], []
        for si, R in enumerate(pb.response_lengths):
            toks = pb.tokens[cu[si]:cu[si + 1]]
            L = int(toks.numel())
            Lp = (L + unit - 1) // unit * unit
            cs = Lp // (2 * cp)
            tok_pad = torch.cat([toks, toks.new_zeros(Lp - L + 1)])
            idx = torch.cat([torch.arange(r * cs, (r + 1) * cs), torch.arange((2 * cp - 1 - r) * cs, (2 * cp - r) * cs)]).to(toks.device)
            mode = self.cfg.cp_attention or ("peer" if self.device.type == "cuda" else "ring")
            if mode == "ring" and self.device.type == "cuda":
                raise RuntimeError("the ring statement of context-parallel attention is a CPU oracle (it materialises "
                                   "the score matrix); use cp_attention='peer' or 'allgather' on a GPU")
            comm = self._cp_comm_for(2 * cs) if mode == "peer" else None

            def attn(layer_idx, q, k, v, L=L, comm=comm, mode=mode):
                if mode == "peer":
                    from ..parallel.cp_peer import peer_attention

                    return peer_attention(q, k.contiguous(), v.contiguous(), comm, L)
                if mode == "allgather":
                    return CP.allgather_attention(q, k, v, g, L)
                return CP.ring_attention(q, k.contiguous(), v.contiguous(), g, L)

            h = self.model(tok_pad[idx], idx, None, attn_fn=attn)
            sel = (idx >= L - R - 1) & (idx <= L - 2)
            lp, en = self.model.log_probs(h[sel], tok_pad[idx + 1][sel], self.cfg.rollout_temperature, with_entropy)
            lps.append(CP.gather_response_with_cp(lp, L, R, g, padded_total_length=Lp))
            ens.append(CP.gather_response_with_cp(en, L, R, g, padded_total_length=Lp) if with_entropy else lp.new_zeros(R))
        return torch.cat(lps), torch.cat(ens)

    def _cp_comm_for(self, rows: int):
        """The NVLink staging buffers of this rank's context-parallel group, (re)made when a sequence needs more local
        rows than they hold.  Collective over the group: every CP rank sees the same sequences in the same order."""
        comm = getattr(self, "cp_comm", None)
        if comm is not None and comm.rows >= rows:
            return comm
        from ..parallel.cp_peer import CPComm

        if comm is not None:
            comm.close()
        tp = self.ps.tp.size
        cap = max(rows, 1 << max(10, (rows - 1).bit_length()))      # grow in powers of two
        self.cp_comm = CPComm(self.ps.cp, self.device, cap, self.mcfg.num_attention_heads // tp,
                              self.mcfg.num_query_groups // tp, self.mcfg.head_dim)
        return self.cp_comm

    def _forward_logp(self, pb, with_entropy: bool):
        if (self.cfg.use_routing_replay or self.cfg.use_rollout_routing_replay) and self.mcfg.is_moe:
            from ..models.moe import RoutingReplay

            RoutingReplay.set_layout(getattr(self, "_cur_ids", None), pb.total_lengths)
        if self.ps.pp.size > 1:
            return self._forward_logp_pp(pb, with_entropy)
        if self.ps.cp.size > 1:
            return self._forward_logp_cp(pb, with_entropy)
        emb = self._embed_multimodal(pb) if getattr(pb, "pixel_patches", None) is not None else None
        h = self.model(pb.tokens, pb.positions, pb.cu_seqlens, max_seqlen=pb.max_seqlen, inputs_embeds=emb)
        hr = h.index_select(0, pb.logit_rows)
        return self.model.log_probs(hr, pb.targets, self.cfg.rollout_temperature, with_entropy)

    def _forward_logp_mtp(self, pb, with_entropy: bool, lb):
        """Main-head log-probs plus the MTP loss of this micro-batch: depth ``k`` at the row that predicts
        response position ``j`` is trained on position ``j + k`` with that position's loss mask; the depths are
        averaged and scaled by ``mtp_loss_scaling_factor`` (Megatron's MTP loss scaling)."""
        from dataclasses import replace as _replace

        from ..models.mtp import mtp_forward

        cfg = self.cfg
        if cfg.mtp_only_training:
            with torch.no_grad():
                h, pre = self.model(pb.tokens, pb.positions, pb.cu_seqlens, max_seqlen=pb.max_seqlen, return_prenorm=True)
        else:
            h, pre = self.model(pb.tokens, pb.positions, pb.cu_seqlens, max_seqlen=pb.max_seqlen, return_prenorm=True)
        lp, en = self.model.log_probs(h.index_select(0, pb.logit_rows), pb.targets, cfg.rollout_temperature, with_entropy)
        depths = mtp_forward(self.model, pre, pb.tokens, pb.positions, pb.cu_seqlens, pb.logit_rows, pb.max_seqlen)
        total = lp.new_zeros(())
        for k, (lpk, valid) in enumerate(depths, start=1):
            mk = _shift_mask(lb.loss_mask, pb.response_lengths, k) * valid.to(lb.loss_mask.dtype)
            lk, _ = L.sft_loss(lpk, _replace(lb, loss_mask=mk, sample_denoms=None), cfg.loss)
            total = total + lk
        return lp, en, total * (cfg.mtp_loss_scaling_factor / max(1, len(depths)))

    def _forward_class_logits(self, pb):
        """One row of class logits per sample, read at its last real token
        (relax/backends/megatron/loss.py sequence-classification loss :1301-1383)."""
        h = self.model(pb.tokens, pb.positions, pb.cu_seqlens, max_seqlen=pb.max_seqlen)
        last = pb.cu_seqlens[1:1 + len(pb.response_lengths)].to(torch.int64) - 1
        return self.model.class_logits(h.index_select(0, last))

    def _forward_values(self, pb):
        """Critic: one scalar per response position (the hidden state that predicts token t+1 also carries V(s_t))."""
        h = self.model(pb.tokens, pb.positions, pb.cu_seqlens, max_seqlen=pb.max_seqlen)
        return self.model.values(h.index_select(0, pb.logit_rows))

    @torch.no_grad()
    def compute_values(self, batch: dict) -> dict:
        """Forward-only critic pass (relax/backends/megatron/loss.py get_values :466-529): per-sample value lists."""
        toks, rl = batch["tokens"], batch["response_lengths"]
        out = [None] * len(toks)
        for mb in self._microbatches([len(t) for t in toks]):
            if not mb:
                self._dummy_forward()
                continue
            pb = self._pack([toks[i] for i in mb], [rl[i] for i in mb])
            v = self._forward_values(pb)
            for i, a in zip(mb, torch.split(v, pb.response_lengths)):
                out[i] = a
        return {"values": out}

    def _microbatches(self, lengths: Sequence[int], for_train: bool = True) -> list[list[int]]:
        cfg = self.cfg
        n = len(lengths)
        if n == 0:
            mbs = []
        elif cfg.use_dynamic_batch_size:
            mbs = balanced_microbatches(list(lengths), cfg.max_tokens_per_gpu)
        else:
            mbs = [list(range(s, min(n, s + cfg.micro_batch_size))) for s in range(0, n, cfg.micro_batch_size)]
        # every data-parallel replica must run the same number of micro-batches
        # (collectives inside the model); short ranks append dummy ones
        cnt = torch.tensor([len(mbs)], device=self.device)
        if self.ps.dp_cp.size > 1:
            dist.all_reduce(cnt, op=dist.ReduceOp.MAX, group=self.ps.dp_cp.group)
        while len(mbs) < int(cnt):
            mbs.append([])
        return mbs

    @torch.no_grad()
    def compute_log_prob(self, batch: dict, tag: str = "actor", with_entropy: bool = False) -> dict:
        """Forward-only pass; returns per-sample lists ``log_probs`` (and ``entropy``)."""
        self.switch_model(tag)
        suspended = None
        if tag not in ("actor", "old_actor") and (self.cfg.use_routing_replay or self.cfg.use_rollout_routing_replay) and self.mcfg.is_moe:
            from ..models.moe import RoutingReplay

            suspended, RoutingReplay.mode = RoutingReplay.mode, None     # reference / teacher route for themselves
        toks, rl = batch["tokens"], batch["response_lengths"]
        mbs = self._microbatches([len(t) for t in toks])
        out_lp = [None] * len(toks)
        out_en = [None] * len(toks)
        for mb in mbs:
            if not mb:
                self._dummy_forward()
                continue
            pb = self._pack_batch(batch, mb)
            self._cur_ids = list(mb)
            lp, en = self._forward_logp(pb, with_entropy)
            for i, a, b in zip(mb, torch.split(lp, pb.response_lengths), torch.split(en, pb.response_lengths)):
                out_lp[i], out_en[i] = a, b
        self.switch_model("actor")
        if suspended is not None:
            from ..models.moe import RoutingReplay

            RoutingReplay.mode = suspended
        res = {"log_probs": out_lp}
        if with_entropy:
            res["entropy"] = out_en
        return res

    @torch.no_grad()
    def compute_topk_log_probs(self, batch: dict, tag: str = "actor", k: int = 0, ids: Optional[Sequence] = None,
                               row_chunk: int = 2048) -> dict:
        """Forward-only pass that reads the distribution on a SET of token ids per response position instead of the
        sampled token only (top-K distillation; relax/utils/opd/opd_utils.py compute_log_probs_on_topk_token_ids
        :1023).  Without ``ids``: this model's own top-``k`` ids per position and their log-probs, ``[R_i, k]`` each.
        With ``ids`` (per sample ``[R_i, K]``, global vocabulary ids, negative = padding): the log-probs of exactly
        those ids (padding gives ``-inf``).  The logits of ``row_chunk`` positions at a time exist in fp32; nothing of
        vocabulary size is kept.  One model-parallel rank per replica (tp = pp = cp = 1)."""
        if self.ps.tp.size > 1 or self.ps.pp.size > 1 or self.ps.cp.size > 1:
            raise NotImplementedError("top-K distillation reads full-vocabulary rows: trainer tp = pp = cp = 1")
        if ids is None and k <= 0:
            raise ValueError("either k > 0 or ids")
        self.switch_model(tag)
        toks = batch["tokens"]
        out_ids, out_lp = [None] * len(toks), [None] * len(toks)
        w = self.model.lm_head_weight()[: self.mcfg.vocab_size].float()
        inv_t = 1.0 / float(self.cfg.rollout_temperature or 1.0)
        for mb in self._microbatches([len(t) for t in toks]):
            if not mb:
                self._dummy_forward()
                continue
            pb = self._pack_batch(batch, mb)
            emb = self._embed_multimodal(pb) if getattr(pb, "pixel_patches", None) is not None else None
            h = self.model(pb.tokens, pb.positions, pb.cu_seqlens, max_seqlen=pb.max_seqlen, inputs_embeds=emb)
            hr = h.index_select(0, pb.logit_rows).float()
            want = None
            if ids is not None:
                rows = [torch.as_tensor(ids[i], dtype=torch.long, device=self.device) for i in mb]
                kmax = max(t.shape[-1] for t in rows)          # union sets differ in width: pad with -1
                want = torch.cat([torch.nn.functional.pad(t, (0, kmax - t.shape[-1]), value=-1) for t in rows])
                if want.shape[0] != hr.shape[0]:
                    raise ValueError("ids must hold one row per response position")
            got_ids, got_lp = [], []
            for a in range(0, hr.shape[0], row_chunk):
                logits = (hr[a:a + row_chunk] @ w.t()) * inv_t
                lse = torch.logsumexp(logits, -1, keepdim=True)
                if want is None:
                    val, idx = logits.topk(k, -1)
                    got_ids.append(idx)
                    got_lp.append(val - lse)
                else:
                    q = want[a:a + row_chunk]
                    lp = logits.gather(-1, q.clamp_min(0)) - lse
                    got_lp.append(lp.masked_fill(q < 0, float("-inf")))
            lp_all = torch.cat(got_lp) if got_lp else hr.new_zeros(0, k)
            for j, (i, piece) in enumerate(zip(mb, torch.split(lp_all, pb.response_lengths))):
                out_lp[i] = piece if ids is None else piece[:, : torch.as_tensor(ids[i]).shape[-1]]
            if want is None:
                for i, piece in zip(mb, torch.split(torch.cat(got_ids), pb.response_lengths)):
                    out_ids[i] = piece
        self.switch_model("actor")
        return {"ids": out_ids if ids is None else list(ids), "log_probs": out_lp}

    # ------------------------------------------------------------------ pipeline parallelism
    def _stage_forward(self, pb, x):
        """This pipeline stage's layers on one packed micro-batch: the first stage embeds the tokens, later stages
        continue from the activations ``x`` received from upstream; the last stage returns the normalised hidden
        states, the others their stage output."""
        if self.model.pre_process:
            return self.model(pb.tokens, pb.positions, pb.cu_seqlens, max_seqlen=pb.max_seqlen)
        return self.model(None, pb.positions, pb.cu_seqlens, hidden_in=x, max_seqlen=pb.max_seqlen)

    def _forward_logp_pp(self, pb, with_entropy: bool):
        """Forward-only pass through the pipeline for one micro-batch; every stage returns the log-probs (the last
        stage computes them and shares them with its pipeline group, so the callers are layout-agnostic).  Sends are
        asynchronous, so consecutive micro-batches overlap across stages."""
        from ..parallel import pp as PP

        g = self.ps.pp
        first, last = g.rank == 0, g.rank == g.size - 1
        x = None if first else PP._recv(g.ranks[g.rank - 1], g.group, self.device, self.model.dtype)
        h = self._stage_forward(pb, x)
        n = int(sum(pb.response_lengths))
        if last:
            lp, en = self.model.log_probs(h.index_select(0, pb.logit_rows), pb.targets, self.cfg.rollout_temperature, with_entropy)
            buf = torch.stack([lp.float(), en.float()])
        else:
            PP._send(h, g.ranks[g.rank + 1], g.group)
            buf = torch.empty(2, n, dtype=torch.float32, device=self.device)
        dist.broadcast(buf, src=g.ranks[-1], group=g.group)
        PP._reap(all_=True)
        return buf[0], buf[1]

    def _sync_tied_embedding_grads(self):
        """With tied input / output embeddings and more than one stage, the first and the last stage each hold a copy
        of the table; their gradients are summed so both copies take the same step."""
        g = self.ps.pp
        if g.size == 1 or not self.mcfg.tie_word_embeddings:
            return
        emb = getattr(getattr(self.model, "embedding", None), "word_embeddings", None)
        if emb is not None:
            grad = emb.weight.main_grad if getattr(emb.weight, "main_grad", None) is not None else emb.weight.grad
        else:       # middle stages take part with zeros (the group has no two-rank sub-group of its own)
            v = (self.mcfg.vocab_size + self.ps.tp.size - 1) // self.ps.tp.size
            grad = torch.zeros(v, self.mcfg.hidden_size, dtype=torch.float32, device=self.device)
        dist.all_reduce(grad, group=g.group)

    def _train_microbatches_pp(self, batch, idx, mbs, metrics, ntok):
        """One optimizer step's micro-batches through the 1F1B schedule.  Every stage holds the whole batch (rows are
        split over data-parallel replicas only), so each packs the micro-batch it works on locally and only
        activations / activation gradients travel."""
        from ..parallel import pp as PP

        cfg, g = self.cfg, self.ps.pp
        last = g.rank == g.size - 1
        dp_cp = self.ps.dp_cp.size
        counter = {"i": 0}

        def forward_step(_mb, x):
            mb = mbs[counter["i"]]
            counter["i"] += 1
            ids = [idx[j] for j in mb]
            if ids:
                pb = self._pack([batch["tokens"][i] for i in ids], [batch["response_lengths"][i] for i in ids])
            else:
                pb = self._pack([[0, 0]], [1])
            self._cur_ids = list(ids)
            h = self._stage_forward(pb, x)
            if not last:
                return h, None
            hr = h.index_select(0, pb.logit_rows)
            if not ids:        # a dummy micro-batch keeps the replicas' schedules aligned; it contributes nothing
                lp, _ = self.model.log_probs(hr, pb.targets, cfg.rollout_temperature, False)
                return h, lp.sum() * 0.0
            lb = self._loss_batch(batch, ids, pb)
            if self.role == "sft":
                lp, _ = self.model.log_probs(hr, pb.targets, cfg.rollout_temperature, False)
                loss, m = L.sft_loss(lp, lb, cfg.loss)
            else:
                lp, en = self.model.log_probs(hr, pb.targets, cfg.rollout_temperature, cfg.compute_entropy)
                loss, m = L.policy_loss(lp, en, lb, cfg.loss)
            ntok.add_(lb.loss_mask.sum() if lb.loss_mask is not None else float(len(ids)))
            for k, v in m.items():
                metrics[k] = metrics.get(k, 0) + v.detach().float()
            return h, loss if cfg.loss.calculate_per_token_loss else loss * (dp_cp / cfg.global_batch_size)

        PP.forward_backward_1f1b(iter(mbs) if g.rank == 0 else None, forward_step, g, self.device, self.model.dtype)
        self._sync_tied_embedding_grads()
        # the loss metrics live on the last stage: share them so every stage reports (and reduces) the same numbers
        obj = [sorted(metrics)] if last else [None]
        dist.broadcast_object_list(obj, src=g.ranks[-1], group=g.group)
        keys = obj[0]
        vec = torch.stack([metrics[k] for k in keys] + [ntok[0]]) if last else torch.zeros(len(keys) + 1, device=self.device)
        dist.broadcast(vec, src=g.ranks[-1], group=g.group)
        metrics.clear()
        metrics.update({k: vec[i] for i, k in enumerate(keys)})
        ntok.copy_(vec[-1:])

    def _dummy_forward(self, backward: bool = False):
        pb = self._pack([[0, 0]], [1])
        if backward:
            if self.role == "critic":
                (self._forward_values(pb).sum() * 0.0).backward()
                return
            lp, en = self._forward_logp(pb, False)
            (lp.sum() * 0.0).backward()
        else:
            with torch.no_grad():
                self._forward_logp(pb, False)

    # ------------------------------------------------------------------ data-parallel split
    def split_for_dp(self, batch: dict) -> dict:
        """Keep this replica's share of a batch that every rank holds in full.
        ``balance_data`` equalises token totals (Karmarkar-Karp), else contiguous."""
        dp, r = self.ps.dp.size, self.ps.dp.rank
        n = len(batch["tokens"])
        if dp == 1:
            return batch
        if self.cfg.balance_data and n % dp == 0:
            idx = karmarkar_karp([len(t) for t in batch["tokens"]], dp, equal_size=True)[r]
        else:
            per = n // dp
            idx = list(range(r * per, (r + 1) * per))
        return {k: ([v[i] for i in idx] if isinstance(v, list) and len(v) == n else v) for k, v in batch.items()}

    # ------------------------------------------------------------------ training
    def forward_log_probs(self, batch: dict) -> dict:
        """The forward-only part of :meth:`train` - reference and old-policy log-probs - on a PART of a rollout batch,
        so that it can run while the rest of the batch is still being generated
        (relax/backends/megatron/actor.py:1103-1125 pulls ``global_batch_size / num_iters_per_train_update`` rows at a
        time for these passes).  The rows come back marked; :meth:`train` then skips the passes.  Parts are joined
        with :func:`concat_batches`.  Routing replay records the routing of the old-policy pass for the optimizer
        passes that follow it directly, which a split pass cannot provide: refused."""
        cfg = self.cfg
        if self.mcfg.is_moe and (cfg.use_routing_replay or cfg.use_rollout_routing_replay):
            raise ValueError("routing replay needs the old-policy pass directly before the optimizer passes: "
                             "use --num-iters-per-train-update 1")
        if "ref" in self.snapshots and (cfg.loss.use_kl_loss or cfg.kl_coef != 0):
            r_ = self.compute_log_prob(batch, "ref", with_entropy=cfg.use_rollout_entropy)
            batch["ref_log_probs"] = r_["log_probs"]
            if cfg.use_rollout_entropy:
                batch["ref_entropy"] = r_["entropy"]
        if cfg.use_rollout_logprobs and batch.get("rollout_log_probs") is not None:
            batch["log_probs"] = [torch.as_tensor(x, dtype=torch.float32, device=self.device) for x in batch["rollout_log_probs"]]
        elif not cfg.loss.true_on_policy:
            tag = "old_actor" if (cfg.keep_old_actor and "old_actor" in self.snapshots) else "actor"
            o_ = self.compute_log_prob(batch, tag, with_entropy=cfg.use_rollout_entropy)
            batch["log_probs"] = o_["log_probs"]
            if cfg.use_rollout_entropy:
                batch["entropy"] = o_["entropy"]
        batch["__forwarded__"] = True
        return batch

    def train(self, rollout_id: int, batch: dict, update_policy: bool = True) -> dict:
        """One rollout's worth of optimizer steps on this replica's samples
        (``batch`` already split for data parallelism).  Returns reduced metrics.  With ``update_policy=False`` only
        the forward passes, advantages and returns are computed (critic warm-up steps of PPO)."""
        cfg, dev = self.cfg, self.device
        t0 = time.perf_counter()
        n = len(batch["tokens"])
        resp = [int(r) for r in batch["response_lengths"]]
        # token-level list fields go to the device ONCE (one flat copy each, then views): the micro-batch loops below
        # read them several times, and a host list -> tensor conversion per sample per pass leaves the device idle
        for key in ("loss_masks", "rollout_log_probs"):
            v = batch.get(key)
            if v is not None and len(v) and not torch.is_tensor(v[0]):
                lens = [len(x) for x in v]
                flat = torch.tensor([y for x in v for y in x], dtype=torch.float32).to(dev, non_blocking=True)
                batch[key] = list(torch.split(flat, lens))
        masks = [torch.as_tensor(m, dtype=torch.float32, device=dev) for m in batch["loss_masks"]]

        forwarded = bool(batch.get("__forwarded__"))      # forward_log_probs() already ran on these rows
        with self.timer.span("ref_log_probs"):
            if not forwarded and "ref" in self.snapshots and (cfg.loss.use_kl_loss or cfg.kl_coef != 0):
                r_ = self.compute_log_prob(batch, "ref", with_entropy=cfg.use_rollout_entropy)
                batch["ref_log_probs"] = r_["log_probs"]
                if cfg.use_rollout_entropy:
                    batch["ref_entropy"] = r_["entropy"]
        r3 = (cfg.use_rollout_routing_replay and self.mcfg.is_moe and batch.get("rollout_routed_experts") is not None)
        if r3:
            from ..models.moe import RoutingReplay

            RoutingReplay.begin_record()          # clears earlier records
            moe_layers = [i for i in range(self.mcfg.num_layers) if self.mcfg.is_moe_layer(i)]
            for sid, routed in enumerate(batch["rollout_routed_experts"]):
                t = torch.as_tensor(routed, dtype=torch.int64, device=dev)        # [positions, L_moe, k]
                for m, layer in enumerate(moe_layers):
                    RoutingReplay.per_sample[(layer, sid)] = t[:, m]
            RoutingReplay.mode = "replay"
        with self.timer.span("old_log_probs"):
            if forwarded:
                pass
            elif cfg.use_rollout_logprobs and batch.get("rollout_log_probs") is not None:
                batch["log_probs"] = [torch.as_tensor(x, dtype=torch.float32, device=dev) for x in batch["rollout_log_probs"]]
            elif not cfg.loss.true_on_policy:
                tag = "old_actor" if (cfg.keep_old_actor and "old_actor" in self.snapshots) else "actor"
                replay = cfg.use_routing_replay and self.mcfg.is_moe and not r3
                if replay:
                    from ..models.moe import RoutingReplay

                    RoutingReplay.begin_record()
                o_ = self.compute_log_prob(batch, tag, with_entropy=cfg.use_rollout_entropy)
                batch["log_probs"] = o_["log_probs"]
                if cfg.use_rollout_entropy:      # relax/backends/megatron/model.py forward_only(with_entropy=args.use_rollout_entropy)
                    batch["entropy"] = o_["entropy"]
                if replay:
                    RoutingReplay.end()
                    RoutingReplay.begin_replay()          # until the end of this rollout's optimizer steps

        seg_all = Segments.from_lengths(resp, device=dev)
        mask_all = torch.cat(masks) if masks else torch.zeros(0, device=dev)
        rewards = torch.as_tensor(batch["rewards"], dtype=torch.float32, device=dev)
        cat = lambda k: torch.cat([torch.as_tensor(x, dtype=torch.float32, device=dev) for x in batch[k]]) \
            if batch.get(k) is not None and len(batch[k]) else None
        adv_stats: dict = {}
        if cfg.compute_advantages_and_returns:
            adv, ret = L.compute_advantages_and_returns(
                cfg.advantage_estimator, rewards, seg_all, mask_all,
                log_probs=cat("log_probs"), ref_log_probs=cat("ref_log_probs"), values=cat("values"),
                kl_coef=cfg.kl_coef, kl_loss_type=cfg.loss.kl_loss_type, gamma=cfg.gamma, lambd=cfg.lambd,
                normalize_advantages=cfg.normalize_advantages, dp_group=self.ps.dp.group, stats_out=adv_stats,
                custom_advantage=(torch.as_tensor(batch["custom_advantages"], dtype=torch.float32, device=dev)
                                  if batch.get("custom_advantages") is not None else None),
            )
            batch["advantages"] = seg_all.split(adv)
            batch["returns"] = seg_all.split(ret)
            if self.replay.wants("advantages", rollout_id) and not (self.ps.dp.size > 1 and cfg.normalize_advantages):
                self.replay.capture("advantages", rollout_id, dict(
                    estimator=cfg.advantage_estimator, rewards=rewards, seg=seg_all, loss_mask=mask_all, log_probs=cat("log_probs"),
                    ref_log_probs=cat("ref_log_probs"), values=cat("values"), kl_coef=cfg.kl_coef, kl_loss_type=cfg.loss.kl_loss_type,
                    gamma=cfg.gamma, lambd=cfg.lambd, normalize_advantages=cfg.normalize_advantages),
                    {"advantages": adv, "returns": ret})
        elif cfg.loss.custom_loss_function is None and self.role == "actor":
            raise ValueError("--disable-compute-advantages-and-returns needs a custom loss function (the policy losses read "
                             "the advantages)")
        opd_metric = None
        if cfg.opd_only_reward and (cfg.opd_kl_coef != 0.0 or cfg.loss.opd_loss_coef != 0.0) and batch.get("advantages") is not None:
            # pure distillation (relax/backends/megatron/loss.py:638-644): the task reward's contribution is removed
            batch["advantages"] = [torch.zeros_like(a) for a in batch["advantages"]]
            batch["returns"] = [torch.zeros_like(r_) for r_ in batch["returns"]]
        if cfg.loss.opd_loss_coef != 0.0 and batch.get("teacher_log_probs") is None and "teacher" in self.snapshots:
            with self.timer.span("teacher_log_probs"):      # loss mode: the term itself is built in the policy loss
                batch["teacher_log_probs"] = self.compute_log_prob(batch, "teacher")["log_probs"]
        if cfg.opd_kl_coef != 0.0 and (batch.get("teacher_log_probs") is not None or "teacher" in self.snapshots):
            from ..algo import opd as OPD

            sel = cfg.opd_token_selection
            kw = dict(kl_type=cfg.opd_kl_type, alpha=cfg.opd_jsd_alpha, norm_mode=cfg.opd_norm_mode,
                      log_prob_min_clamp=cfg.opd_log_prob_min_clamp)
            if sel == "sampled_token":
                with self.timer.span("teacher_log_probs"):
                    if batch.get("teacher_log_probs") is None:
                        batch["teacher_log_probs"] = self.compute_log_prob(batch, "teacher")["log_probs"]
                student = batch.get("log_probs") or self.compute_log_prob(batch, "actor")["log_probs"]
                sig = [OPD.per_token_signal("sampled_token", student_lp=torch.as_tensor(a, dtype=torch.float32, device=dev),
                                            teacher_lp=torch.as_tensor(b, dtype=torch.float32, device=dev), **kw)
                       for a, b in zip(student, batch["teacher_log_probs"])]
            else:
                # both distributions on a set of K ids per position (relax/utils/opd/opd_utils.py:1275-1420): the set is
                # the student's top-K, the teacher's, or their union (rows of different width, padded and masked)
                if "teacher" not in self.snapshots:
                    raise ValueError(f"--opd-token-selection {sel} needs the teacher's distribution: an in-process teacher "
                                     "(--opd-teacher-load); remote teachers return the sampled token's log-prob only")
                k = cfg.opd_log_prob_top_k
                if k <= 0:
                    raise ValueError(f"--opd-token-selection {sel} needs --opd-log-prob-top-k > 0")
                with self.timer.span("teacher_log_probs"):
                    own_s = self.compute_topk_log_probs(batch, "actor", k=k) if sel in ("student_topk", "union") else None
                    own_t = self.compute_topk_log_probs(batch, "teacher", k=k) if sel in ("teacher_topk", "union") else None
                    lengths = None
                    if sel == "student_topk":
                        ids = own_s["ids"]
                    elif sel == "teacher_topk":
                        ids = own_t["ids"]
                    else:
                        pairs = [OPD.union_ids(a, b) for a, b in zip(own_s["ids"], own_t["ids"])]
                        lengths = [n for _, n in pairs]
                        col = lambda u, n: torch.arange(u.shape[-1], device=u.device)[None, :] < n[:, None]
                        ids = [u.masked_fill(~col(u, n), -1) for u, n in pairs]
                    s_lp = own_s["log_probs"] if sel == "student_topk" else self.compute_topk_log_probs(batch, "actor", ids=ids)["log_probs"]
                    t_lp = own_t["log_probs"] if sel == "teacher_topk" else self.compute_topk_log_probs(batch, "teacher", ids=ids)["log_probs"]
                sig = [OPD.per_token_signal(sel, student_topk_lp=a, teacher_topk_lp=b, k_lengths=(lengths[i] if lengths else None), **kw)
                       for i, (a, b) in enumerate(zip(s_lp, t_lp))]
                batch["opd_topk_token_ids"] = ids
            batch["advantages"] = OPD.apply_to_advantages(list(batch["advantages"]), sig, cfg.opd_kl_coef, cfg.opd_per_token_clip)
            tot = sum(float((d * m).sum()) for d, m in zip(sig, masks))
            opd_metric = tot / max(1.0, float(mask_all.sum()))

        from ..data.rollout_log import log_rollout_data

        rollout_stats = log_rollout_data(batch, self.ps.dp.group if self.ps.dp.size > 1 else None,
                                         device=dev if (dist.is_initialized() and dist.get_backend() == "nccl") else "cpu")
        dp = self.ps.dp.size
        per_step = max(1, cfg.global_batch_size // dp)
        steps = max(1, math.ceil(n / per_step)) if n else 1
        nsteps = torch.tensor([steps], device=dev)
        if self.ps.dp_cp.size > 1:
            dist.all_reduce(nsteps, op=dist.ReduceOp.MAX, group=self.ps.dp_cp.group)
        agg: dict[str, torch.Tensor] = {}
        last_norm = 0.0
        for s in range(int(nsteps) if update_policy else 0):
            idx = list(range(s * per_step, min(n, (s + 1) * per_step)))
            with self.timer.span("train_step"):
                self._cur_rollout, self._cur_step = rollout_id, s
                m, last_norm = self._train_step(batch, idx)
            if cfg.ci is not None and (cfg.ci.enabled or cfg.ci.save_grad_norm or cfg.ci.load_grad_norm):
                from . import ci_utils as CI

                self._ci_steps = getattr(self, "_ci_steps", 0)
                CI.check_first_step_kl(cfg.ci, m, s, self._ci_steps)
                CI.save_or_check_grad_norm(cfg.ci, self.role, rollout_id, s, last_norm, self.ps.global_rank)
                self._ci_steps += 1
            for k, v in m.items():
                agg[k] = agg.get(k, 0) + v / int(nsteps)
        if (cfg.use_routing_replay or r3) and self.mcfg.is_moe:
            from ..models.moe import RoutingReplay

            RoutingReplay.end()
        out = {k: float(v) for k, v in agg.items()}
        if opd_metric is not None:
            out["opd_kl"] = opd_metric
        out.update({k: float(v) for k, v in adv_stats.items()})
        out.update(rollout_stats)
        out["grad_norm"] = last_norm
        out["train_time"] = time.perf_counter() - t0
        return out

    def _loss_batch(self, batch, idx, pb) -> L.LossBatch:
        dev = self.device
        f = lambda key: torch.cat([torch.as_tensor(batch[key][i], dtype=torch.float32, device=dev) for i in idx]) \
            if batch.get(key) is not None else None
        seg = Segments.from_lengths(pb.response_lengths, device=dev)
        denoms = None
        if batch.get("sample_index_mask_sums") is not None:
            from ..algo.ppo_utils import to_device_async

            denoms = to_device_async(torch.tensor([float(batch["sample_index_mask_sums"][i]) for i in idx], dtype=torch.float32), dev)
        extras = {}
        if self.cfg.loss.opd_loss_coef != 0.0 and batch.get("teacher_log_probs") is not None:
            extras["teacher_log_probs"] = f("teacher_log_probs")
        return L.LossBatch(seg=seg, loss_mask=f("loss_masks"), advantages=f("advantages"),
                           old_log_probs=f("log_probs"), ref_log_probs=f("ref_log_probs"),
                           rollout_log_probs=f("rollout_log_probs"), returns=f("returns"), values=f("values"),
                           sample_denoms=denoms, extras=extras)

    def _train_step(self, batch, idx):
        cfg, ps = self.cfg, self.ps
        opt = self.optimizer
        self.switch_model("actor")
        opt.zero_grad()
        lens = [len(batch["tokens"][i]) for i in idx]
        mbs = self._microbatches(lens)
        dp_cp = ps.dp_cp.size
        metrics: dict[str, torch.Tensor] = {}
        ntok = torch.zeros(1, device=self.device)
        if ps.pp.size > 1:
            if self.role not in ("actor", "sft") or cfg.loss.custom_loss_function is not None or self.mcfg.mtp_num_layers > 0:
                raise NotImplementedError("pipeline parallelism covers the policy and SFT losses of the plain decoder")
            self._train_microbatches_pp(batch, idx, mbs, metrics, ntok)
            mbs = []
        for mb in mbs:
            if not mb:
                self._dummy_forward(backward=True)
                continue
            ids = [idx[j] for j in mb]
            self._cur_ids = list(ids)
            pb = self._pack_batch(batch, ids)
            lb = self._loss_batch(batch, ids, pb)
            use_mtp = (cfg.enable_mtp_training or cfg.mtp_only_training) and self.mcfg.mtp_num_layers > 0
            if self.role == "critic":
                loss, m = L.value_loss(self._forward_values(pb), lb, cfg.loss)
            elif self.role == "seq_cls":
                labels = torch.as_tensor([batch["labels"][i] for i in ids], device=self.device)
                loss, m = L.seq_cls_loss(self._forward_class_logits(pb), labels, cfg.problem_type or "single_label_classification",
                                         cfg.classification_threshold)
            elif use_mtp:
                lp, en, mtp = self._forward_logp_mtp(pb, cfg.compute_entropy and self.role != "sft", lb)
                if cfg.mtp_only_training:
                    loss, m = mtp, {"loss": mtp.detach()}
                else:
                    loss, m = L.sft_loss(lp, lb, cfg.loss) if self.role == "sft" else L.policy_loss(lp, en, lb, cfg.loss)
                    loss = loss + mtp
                m["mtp_loss"] = mtp.detach()
            elif self.role == "sft":
                lp, _ = self._forward_logp(pb, False)
                loss, m = L.sft_loss(lp, lb, cfg.loss)
            elif cfg.loss.custom_loss_function is not None:
                lp, en = self._forward_logp(pb, cfg.compute_entropy)
                loss, m = cfg.loss.custom_loss_function(lp, en, lb, cfg.loss)
            else:
                lp, en = self._forward_logp(pb, cfg.compute_entropy)
                loss, m = L.policy_loss(lp, en, lb, cfg.loss)
                if self.replay.wants("loss", self._cur_rollout, self._cur_step) and ps.cp.size == 1:
                    # what the loss consumed and produced (post-forward statistics, no logits, no weights)
                    self.replay.capture("loss", self._cur_rollout, dict(log_probs=lp.detach(), entropy=en.detach(), batch=lb, cfg=cfg.loss),
                                        {"loss": loss.detach(), "metrics": m}, step_id=self._cur_step)
            if self.mcfg.dsa_topk > 0:
                from ..models.hybrid import collect_indexer_loss

                aux = collect_indexer_loss(self.model)
                if aux is not None:     # per micro-batch mean; weighted like one sample per packed sequence
                    loss = loss + aux * (self.mcfg.dsa_indexer_loss_coef * len(ids))
                    m["indexer_loss"] = aux.detach() * len(ids)
            ntok += lb.loss_mask.sum() if lb.loss_mask is not None else float(len(ids))
            if cfg.loss.calculate_per_token_loss:
                scaled = loss
            else:
                scaled = loss * (dp_cp / cfg.global_batch_size)
            scaled.backward()
            for k, v in m.items():
                metrics[k] = metrics.get(k, 0) + v.detach().float()
        gscale = 1.0
        if cfg.loss.calculate_per_token_loss:
            tot = ntok.clone()
            if dp_cp > 1:
                dist.all_reduce(tot, group=ps.dp_cp.group)
            gscale = dp_cp / float(tot.clamp_min(1))
        norm, skipped = opt.step(grad_scale=gscale)
        if self.mcfg.moe_router_bias:      # auxiliary-loss-free balancing: token counts of this step, all replicas
            for mod in self.model.modules():
                if hasattr(mod, "update_router_bias"):
                    mod.update_router_bias(self.mcfg.moe_router_bias_update_rate, ps.dp_cp.group if dp_cp > 1 else None)
        # metrics: sum over samples -> mean over the global batch
        keys = sorted(metrics)
        if keys:
            vec = torch.stack([metrics[k] for k in keys])
        else:
            vec = torch.zeros(0, device=self.device)
        if cfg.loss.calculate_per_token_loss:
            denom = ntok.clone()
        else:
            denom = torch.tensor([float(len(idx))], device=self.device)
        pack = torch.cat([vec, denom])
        if dp_cp > 1:
            # every replica must contribute the same keys; keys depend only on the config
            dist.all_reduce(pack, group=ps.dp_cp.group)
        d = pack[-1].clamp_min(1)
        out = {k: pack[i] / d for i, k in enumerate(keys)}
        return out, norm

    def train_critic(self, rollout_id: int, batch: dict) -> dict:
        """PPO critic update (relax/backends/megatron/actor.py train_critic :844-888): ``batch`` carries the
        rollout-time ``values`` and the GAE ``returns`` computed with them; clipped value loss."""
        assert self.role == "critic"
        return self._optimizer_steps(batch)

    def train_seq_cls(self, batch: dict) -> dict:
        """Sequence-classification fine-tuning: cross entropy of the class head at each sample's last token
        against ``batch["labels"]``; metrics carry the accuracy."""
        assert self.role == "seq_cls" and self.mcfg.num_classes > 0
        return self._optimizer_steps(batch)

    @torch.no_grad()
    def predict_classes(self, batch: dict) -> list:
        out = [None] * len(batch["tokens"])
        lens = [len(t) for t in batch["tokens"]]
        for mb in self._microbatches(lens, for_train=False):
            if not mb:
                self._dummy_forward()
                continue
            pb = self._pack([batch["tokens"][i] for i in mb], [batch["response_lengths"][i] for i in mb])
            for i, row in zip(mb, self._forward_class_logits(pb)):
                out[i] = row
        return out

    def train_sft(self, batch: dict) -> dict:
        """Supervised step(s): next-token cross entropy over the positions with ``loss_masks`` 1
        (relax/backends/megatron/loss.py sft_loss_function :1247-1298).  ``tokens`` are prompt+response,
        ``response_lengths`` the trained suffix of each sample."""
        assert self.role == "sft"
        return self._optimizer_steps(batch)

    def _optimizer_steps(self, batch: dict) -> dict:
        cfg, dev = self.cfg, self.device
        n = len(batch["tokens"])
        per_step = max(1, cfg.global_batch_size // self.ps.dp.size)
        nsteps = torch.tensor([max(1, math.ceil(n / per_step)) if n else 1], device=dev)
        if self.ps.dp_cp.size > 1:
            dist.all_reduce(nsteps, op=dist.ReduceOp.MAX, group=self.ps.dp_cp.group)
        agg: dict = {}
        norm = 0.0
        for s_ in range(int(nsteps)):
            idx = list(range(s_ * per_step, min(n, (s_ + 1) * per_step)))
            m, norm = self._train_step(batch, idx)
            for k, v in m.items():
                agg[k] = agg.get(k, 0) + v / int(nsteps)
        out = {k: float(v) for k, v in agg.items()}
        out["grad_norm"] = norm
        return out

    @torch.no_grad()
    def evaluate_ppl(self, batch: dict) -> dict:
        """Token-level negative log-likelihood and perplexity over the masked positions (SFT eval)."""
        lps = self.compute_log_prob(batch)["log_probs"]
        tot = torch.zeros(2, device=self.device, dtype=torch.float64)
        for lp, m in zip(lps, batch["loss_masks"]):
            m = torch.as_tensor(m, dtype=torch.float32, device=self.device)
            tot[0] += -(lp.float() * m).sum()
            tot[1] += m.sum()
        if self.ps.dp_cp.size > 1:
            dist.all_reduce(tot, group=self.ps.dp_cp.group)
        nll = float(tot[0] / tot[1].clamp_min(1))
        return {"eval/nll": nll, "eval/ppl": math.exp(min(nll, 50.0)), "eval/tokens": float(tot[1])}

    # ------------------------------------------------------------------ misc
    def after_train(self):
        self.weight_version += 1
        if self.cfg.keep_old_actor:
            self.backup("old_actor")

    def named_local_params(self, merged: bool = True):
        """(megatron-style name, tensor) for every local parameter, actor weights.  With LoRA: the merged weights
        (default) or, ``merged=False``, the frozen base weights and the factors as they are (adapter-mode sync)."""
        self.switch_model("actor")
        if self.cfg.lora is not None and merged:
            from .lora import merged_named_params

            return merged_named_params(self.model)   # merged-weights sync: the engine sees a plain model
        return list(self.model.named_parameters())

    def sleep(self):
        if self.optimizer is not None:
            self.optimizer.offload_state()

    def wake_up(self):
        if self.optimizer is not None:
            self.optimizer.onload_state()
