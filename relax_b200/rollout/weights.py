"""Parameter buffers and model forward of the rollout engine.

Layout ("rollout layout", one TP shard per rank, all in ONE flat buffer so the
weight-sync kernel writes into a single registered region):

* ``layers.{i}.qkv``      ``[(nq + 2 nkv) * hd, H]`` rows ordered ``[q heads | k heads | v heads]``
* ``layers.{i}.o``        ``[H, nq * hd]``
* ``layers.{i}.gate_up``  ``[2 F, H]`` rows ``[gate | up]``
* ``layers.{i}.down``     ``[H, F]``
* ``layers.{i}.input_norm / post_norm / q_norm / k_norm``
* ``embed [V_l, H]``, ``lm_head [V_l, H]`` (aliases ``embed`` when tied), ``final_norm``
* MoE layers: ``router [E, H]``, ``experts_gate_up [E_l, 2F, H]``, ``experts_down [E_l, H, F]``

The HF/serving order of q|k|v differs from the trainer's per-group interleave;
the permutation is applied by the weight-sync path
(:mod:`relax_b200.weight_sync`).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..models.config import ModelConfig
from ..parallel.state import GroupInfo


GDN_CONV_KERNEL = 4      # taps of the Gated-DeltaNet depth-wise convolution (relax_b200/models/gdn.py)


def rollout_param_shapes(cfg: ModelConfig, tp: int, ep: int = 1, mtp: bool = False) -> dict:
    """``mtp``: the buffer also holds the first multi-token-prediction block (draft model of speculative decoding) -
    its transformer layer as layer ``num_layers`` and ``mtp.enorm / mtp.hnorm / mtp.eh_proj / mtp.final_norm`` - AFTER
    everything else, so that the offsets of the policy's own tensors do not depend on the switch."""
    hd, H = cfg.head_dim, cfg.hidden_size
    nq, nkv = cfg.num_attention_heads // tp, cfg.num_query_groups // tp
    v_pad = (cfg.vocab_size + tp - 1) // tp * tp
    shapes = {"embed": (v_pad // tp, H)}

    def layer(i):
        from ..models.hybrid import mixer_kind

        p = f"layers.{i}."
        shapes[p + "input_norm"] = (H,)
        if mixer_kind(cfg, i) == "gdn":
            hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
            kd, vd = hk * d, hv * d
            shapes[p + "gdn_qkvz"] = (2 * kd + 2 * vd, H)
            shapes[p + "gdn_ba"] = (2 * hv, H)
            shapes[p + "gdn_conv"] = (2 * kd + vd, GDN_CONV_KERNEL)
            shapes[p + "gdn_dt_bias"], shapes[p + "gdn_A_log"], shapes[p + "gdn_norm"] = (hv,), (hv,), (d,)
            shapes[p + "gdn_out"] = (H, vd)
            return mlp(i, p)
        if mixer_kind(cfg, i) == "dsa":          # multi-head latent attention, sparse when dsa_topk > 0
            nh, nope, rope, kvl, vh = cfg.num_attention_heads, cfg.dsa_nope, cfg.dsa_rope, cfg.dsa_kv_lora, cfg.dsa_v_head
            shapes[p + "mla_q_down"], shapes[p + "mla_q_norm"] = (cfg.dsa_q_lora, H), (cfg.dsa_q_lora,)
            shapes[p + "mla_q_up"] = (nh * (nope + rope), cfg.dsa_q_lora)
            shapes[p + "mla_kv_down"], shapes[p + "mla_kv_norm"] = (kvl + rope, H), (kvl,)
            shapes[p + "mla_kv_up"] = (nh * (nope + vh), kvl)
            shapes[p + "mla_o"] = (H, nh * vh)
            if cfg.dsa_topk > 0:
                shapes[p + "idx_wq"] = (cfg.dsa_index_heads * cfg.dsa_index_dim, H)
                shapes[p + "idx_wk"] = (cfg.dsa_index_dim, H)
                shapes[p + "idx_w"] = (cfg.dsa_index_heads, H)
            return mlp(i, p)
        shapes[p + "qkv"] = ((nq + 2 * nkv) * hd, H)
        if cfg.attention_output_gate:
            shapes[p + "attn_gate"] = (nq * hd, H)       # one gate row per query feature (sigmoid on the attention output)
        if cfg.qkv_bias:
            shapes[p + "qkv_bias"] = ((nq + 2 * nkv) * hd,)
        if cfg.qk_layernorm:
            shapes[p + "q_norm"] = (hd,)
            shapes[p + "k_norm"] = (hd,)
        shapes[p + "o"] = (H, nq * hd)
        mlp(i, p)

    def mlp(i, p):
        shapes[p + "post_norm"] = (H,)
        if cfg.sandwich_norm:          # GLM-4: the block outputs are normed before they join the residual stream
            shapes[p + "post_attn_norm"] = (H,)
            shapes[p + "post_mlp_norm"] = (H,)
        if cfg.is_moe_layer(i):
            el = cfg.num_experts // ep
            shapes[p + "router"] = (cfg.num_experts, H)
            if cfg.moe_router_bias:
                shapes[p + "router_bias"] = (cfg.num_experts,)
            if cfg.moe_shared_expert_ffn > 0:
                shapes[p + "shared_gate_up"] = (2 * cfg.moe_shared_expert_ffn, H)
                shapes[p + "shared_down"] = (H, cfg.moe_shared_expert_ffn)
                if cfg.moe_shared_expert_gate:
                    shapes[p + "shared_gate"] = (1, H)
            shapes[p + "experts_gate_up"] = (el, 2 * cfg.moe_ffn_hidden_size, H)
            shapes[p + "experts_down"] = (el, H, cfg.moe_ffn_hidden_size)
        else:
            F = cfg.ffn_hidden_size // tp
            shapes[p + "gate_up"] = (2 * F, H)
            shapes[p + "down"] = (H, F)

    for i in range(cfg.num_layers):
        layer(i)
    shapes["final_norm"] = (H,)
    if not cfg.tie_word_embeddings:
        shapes["lm_head"] = (v_pad // tp, H)
    if mtp:
        layer(cfg.num_layers)
        shapes["mtp.enorm"], shapes["mtp.hnorm"], shapes["mtp.final_norm"] = (H,), (H,), (H,)
        shapes["mtp.eh_proj"] = (H, 2 * H)
    return shapes


def rollout_layout(cfg: ModelConfig, tp: int, ep: int = 1, mtp: bool = False):
    """``(shapes, element offsets, total elements)`` of one rank's flat parameter buffer.  A pure function of the
    configuration, so a trainer rank can address tensors inside a rollout rank's buffer without asking it."""
    shapes = rollout_param_shapes(cfg, tp, ep, mtp)
    offsets, n = {}, 0
    for k, s in shapes.items():
        offsets[k] = n
        n += (math.prod(s) + 127) // 128 * 128
    return shapes, offsets, n


class RolloutWeights:
    def __init__(self, cfg: ModelConfig, tp_size: int, tp_rank: int, device, dtype, ep_size: int = 1, ep_rank: int = 0,
                 memory_saver: bool = False, shared_path: Optional[str] = None, mtp: bool = False):
        if (cfg.linear_attention_freq > 0 or cfg.attention_output_gate or cfg.dsa_topk > 0 or cfg.multi_latent_attention) \
                and (tp_size > 1 or ep_size > 1 or mtp):
            raise NotImplementedError("stacks with Gated-DeltaNet, gated-attention or latent-attention (MLA / DSA) layers run on "
                                      "one rank per engine, without speculative decoding")
        if cfg.attention_output_gate and cfg.qkv_bias:
            raise NotImplementedError("gated attention with a QKV bias")
        self.cfg, self.tp_size, self.tp_rank = cfg, tp_size, tp_rank
        self.ep_size, self.ep_rank = ep_size, ep_rank
        self.ep_group: Optional[GroupInfo] = None     # the engine's expert-parallel group (set by the engine when ep > 1)
        # routing capture (R3: the trainer replays the rollout's expert choices): when a list, every MoE layer appends
        # its top-k expert ids ``[T, k]`` of the current forward, in layer order
        self.routing_capture: Optional[list] = None
        self.moe_layers = [i for i in range(cfg.num_layers) if cfg.is_moe_layer(i)]
        self.device, self.dtype = torch.device(device), dtype
        self.seq_ctx: Optional[dict] = None      # what the rows of the running forward are (read by the GDN layers)
        self.mtp = bool(mtp)          # the buffer also holds the first MTP block (draft model of speculative decoding)
        if self.mtp and cfg.mtp_num_layers < 1:
            raise ValueError("speculative decoding drafts with the model's multi-token-prediction block; this model has none")
        self.shapes, self.offsets, self.numel = rollout_layout(cfg, tp_size, ep_size, self.mtp)
        # CPU only: back the buffer by a shared-memory file so that other processes can map and write it (the CPU
        # stand-in for a peer mapping of device memory; see weight_sync/peer_push.py)
        self.shared_path = shared_path
        self.flat = None
        self.p: dict[str, torch.Tensor] = {}
        self.lora: dict[str, torch.Tensor] = {}       # adapter-mode serving: see enable_lora()
        self.lora_scale = 0.0
        self.memory_saver = memory_saver
        self._buf = None
        self.resume()
        self.v_local = self.shapes["embed"][0]
        self.vocab_start = tp_rank * self.v_local

    def resume(self):
        if self.memory_saver:
            if self._buf is not None:
                self._buf.resume()     # same addresses, zero-filled: the next weight sync rewrites everything
                return
            from ..utils.memory_saver import PausableBuffer

            self._buf = PausableBuffer(self.numel * torch.empty(0, dtype=self.dtype).element_size(), self.device)
            self.flat = self._buf.tensor((self.numel,), self.dtype)
        elif self.flat is not None:
            return
        elif self.shared_path is not None and self.device.type == "cpu":
            self.flat = torch.from_file(self.shared_path, shared=True, size=self.numel, dtype=self.dtype)
            self.flat.zero_()
        else:
            self.flat = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
        self.p = {k: self.flat[o:o + math.prod(self.shapes[k])].view(self.shapes[k]) for k, o in self.offsets.items()}
        if self.cfg.tie_word_embeddings:
            self.p["lm_head"] = self.p["embed"]
        self.p.update(self.lora)

    def enable_lora(self, rank: int, scale: float, targets=("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2")):
        """Adapter-mode serving: the base weights stay as synced once and every adapted linear adds
        ``scale * B (A x)`` at run time, so a weight sync moves the factors only.  The factors live outside the flat
        buffer (they are small and survive release / resume) under ``<weight name>.lora_A`` / ``.lora_B``; ``B`` starts
        at zero, i.e. the model is the base model until the first adapter sync."""
        from ..weight_sync.plan import _ADAPTED

        self.lora_scale = float(scale)
        for name, shape in self.shapes.items():
            leaf = name.rsplit(".", 1)[-1]
            if not name.startswith("layers.") or leaf not in _ADAPTED or _ADAPTED[leaf][0] not in targets:
                continue
            out_f, in_f = shape
            self.lora[name + ".lora_A"] = torch.zeros(rank, in_f, dtype=self.dtype, device=self.device)
            self.lora[name + ".lora_B"] = torch.zeros(out_f, rank, dtype=self.dtype, device=self.device)
        self.p.update(self.lora)

    def _lora_add(self, name: str, x, y):
        a = self.lora.get(name + ".lora_A")
        if a is None:
            return y
        return y + ops.linear(ops.linear(x, a), self.lora[name + ".lora_B"]) * self.lora_scale

    def release(self):
        if self.memory_saver:
            self._buf.pause()          # views in ``self.p`` keep their addresses and must not be used until resume()
            return
        self.flat, self.p = None, {}

    # ------------------------------------------------------------------ model pieces
    def _embed(self, tokens, tp: GroupInfo):
        w = self.p["embed"]
        if tp.size == 1:
            return w[tokens]
        loc = tokens - self.vocab_start
        ok = (loc >= 0) & (loc < self.v_local)
        e = w[torch.where(ok, loc, torch.zeros_like(loc))] * ok[:, None].to(w.dtype)
        dist.all_reduce(e, group=tp.group)
        return e

    def _allreduce(self, x, tp: GroupInfo):
        if tp.size > 1:
            dist.all_reduce(x, group=tp.group)
        return x

    def _logits(self, h, tp: GroupInfo):
        z = ops.linear(h, self.p["lm_head"])
        if not z.is_cuda:
            z = z.float()       # the sampling kernel reads bf16 rows directly; the CPU statement wants fp32
        if tp.size > 1:
            out = torch.empty(tp.size * z.shape[0], z.shape[1], dtype=z.dtype, device=z.device)
            dist.all_gather_into_tensor(out, z.contiguous(), group=tp.group)
            z = out.view(tp.size, z.shape[0], z.shape[1]).permute(1, 0, 2).reshape(z.shape[0], -1)
        return z

    def _mlp(self, i, x, tp):
        p, cfg = self.p, self.cfg
        pre = f"layers.{i}."
        if pre + "router" in p:
            logits = torch.nn.functional.linear(x.float(), p[pre + "router"].float())
            from ..models.moe import route_tokens

            w, idx, _ = route_tokens(logits, cfg, p.get(pre + "router_bias"))
            if self.routing_capture is not None:
                self.routing_capture.append(idx)
            out = torch.zeros_like(x, dtype=torch.float32)
            if pre + "shared_gate_up" in p and self.ep_rank == 0:     # summed over the EP ranks afterwards: one rank adds it
                sh = ops.linear(ops.swiglu(ops.linear(x, p[pre + "shared_gate_up"])), p[pre + "shared_down"]).float()
                if pre + "shared_gate" in p:
                    sh = sh * torch.sigmoid(ops.linear(x, p[pre + "shared_gate"]).float())
                out += sh
            # every routed (token, slot) pair through the grouped expert GEMMs in one go: rows of experts that live on
            # another EP rank are parked (no math), the per-token sum over the k slots applies the gate weights
            from ..models.moe import grouped_swiglu_mlp

            el = p[pre + "experts_gate_up"].shape[0]
            T, k = idx.shape
            rows = x.repeat_interleave(k, 0)                        # row t*k + j = token t, slot j
            y = grouped_swiglu_mlp(rows, idx.reshape(-1) - self.ep_rank * el, p[pre + "experts_gate_up"],
                                   p[pre + "experts_down"], skip_foreign=True)
            out += (y.float().view(T, k, -1) * w.float().unsqueeze(-1)).sum(1)
            return out.to(x.dtype), (self.ep_group if self.ep_size > 1 else None)
        if self.lora:       # adapter-mode serving: the factors' products join before the activation / before the reduction
            a = ops.swiglu(self._lora_add(pre + "gate_up", x, ops.linear(x, p[pre + "gate_up"])))
            return self._lora_add(pre + "down", a, ops.linear(a, p[pre + "down"])), (tp if tp.size > 1 else None)
        a = ops.linear_swiglu(x, p[pre + "gate_up"])
        return ops.linear(a, p[pre + "down"]), (tp if tp.size > 1 else None)

    def _fused(self, tp: GroupInfo, rows: int, n: int):
        """The symmetric-memory communicator of ``tp`` when the fused GEMM + all-reduce + residual +
        RMSNorm kernel can take a call of this size, else None (NCCL statement)."""
        from ..ops import fused_comm

        comm = fused_comm.comm_of(tp)
        if comm is None or not comm.supports("gemm_ar_add_rmsnorm") or not comm.fits(rows, n):
            return None
        return comm

    # ------------------------------------------------------------------ Gated DeltaNet layers (hybrid stacks)
    def _gdn(self, i, x):
        """The GDN token mixer on rows (relax_b200/models/gdn.py GatedDeltaNet.forward), with the per-sequence state
        that incremental decoding needs: the last ``K - 1`` pre-convolution rows and the recurrent matrix
        ``S [hv, dk, dv]`` (fp32).  ``self.seq_ctx`` says what the rows are: whole sequences (``mode = "prefill"``,
        ``cu`` boundaries; the final states are left in ``ctx["out"][i]``, one pair per sequence) or one new token per
        sequence (``mode = "decode"``, ``ctx["state"][i] = [conv [B, K-1, C], S [B, hv, dk, dv]]``, updated in place)."""
        import torch.nn.functional as F

        from ..models.gdn import causal_conv1d_varlen, gated_delta_rule_chunked

        cfg, p, ctx = self.cfg, self.p, self.seq_ctx
        pre = f"layers.{i}."
        hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
        kd, vd, K = hk * d, hv * d, GDN_CONV_KERNEL
        T = x.shape[0]
        qkvz = ops.linear(x, p[pre + "gdn_qkvz"])
        ba = ops.linear(x, p[pre + "gdn_ba"]).float()
        raw, z = qkvz[:, : 2 * kd + vd], qkvz[:, 2 * kd + vd:]
        w = p[pre + "gdn_conv"]
        if ctx["mode"] == "prefill":
            qkv = causal_conv1d_varlen(raw, w, ctx["cu_t"])
        else:
            conv, _ = ctx["state"][i]
            win = torch.cat([conv.to(raw.dtype), raw[:, None]], 1)                   # [B, K, C]
            qkv = F.silu((win.float() * w.float().t()[None]).sum(1)).to(raw.dtype)
            ctx["state"][i][0] = win[:, 1:]
        q = F.normalize(qkv[:, :kd].reshape(T, hk, d).float(), dim=-1)
        k = F.normalize(qkv[:, kd:2 * kd].reshape(T, hk, d).float(), dim=-1)
        v = qkv[:, 2 * kd:].reshape(T, hv, d)
        if hv // hk > 1:
            q, k = q.repeat_interleave(hv // hk, 1), k.repeat_interleave(hv // hk, 1)
        beta = torch.sigmoid(ba[:, :hv])
        g = -p[pre + "gdn_A_log"].float().exp() * F.softplus(ba[:, hv:] + p[pre + "gdn_dt_bias"].float())
        if ctx["mode"] == "prefill":
            outs, fin = [], []
            for a, b in zip(ctx["cu"], ctx["cu"][1:]):
                o_, S = gated_delta_rule_chunked(q[a:b], k[a:b], v[a:b], g[a:b], beta[a:b])
                tail = raw[max(a, b - (K - 1)):b]
                if tail.shape[0] < K - 1:
                    tail = torch.cat([tail.new_zeros(K - 1 - tail.shape[0], tail.shape[1]), tail])
                outs.append(o_)
                fin.append([tail.clone(), S])
            ctx["out"][i] = fin
            o = torch.cat(outs) if outs else q.new_zeros(0, hv, d)
        else:
            S = ctx["state"][i][1]
            S = S * g.exp()[:, :, None, None]
            u = (v.float() - torch.einsum("bhkv,bhk->bhv", S, k)) * beta[..., None]
            S = S + torch.einsum("bhk,bhv->bhkv", k, u)
            o = torch.einsum("bhkv,bhk->bhv", S, q * d ** -0.5)
            ctx["state"][i][1] = S
        o = ops.rmsnorm(o.to(x.dtype), p[pre + "gdn_norm"], cfg.rms_norm_eps) * F.silu(z.reshape(T, hv, d))
        return ops.linear(o.reshape(T, vd), p[pre + "gdn_out"])

    # ------------------------------------------------------------------ latent attention layers (MLA, sparse = DSA)
    def _mla(self, i, x):
        """Multi-head latent attention on rows (relax_b200/models/dsa.py DSAAttention, absorbed form) with the cache that
        incremental decoding needs: per sequence the latent rows ``[kv_lora | rope]`` of every fed token and, for the
        sparse form, its indexer keys.  ``seq_ctx``: ``mode = "prefill"`` (whole sequences; the caches of every sequence
        are left in ``ctx["out"][i]`` with room for ``ctx["cap"][j]`` rows) or ``"decode"`` (one new token per sequence:
        ``ctx["cache"][i][j] = [latent rows, indexer keys]`` holding ``ctx["lens"][j]`` rows; the new row is appended)."""
        import torch.nn.functional as F

        from ..models import dsa as D

        cfg, p, ctx = self.cfg, self.p, self.seq_ctx
        pre = f"layers.{i}."
        H, nope, rope, kvl, vh = cfg.num_attention_heads, cfg.dsa_nope, cfg.dsa_rope, cfg.dsa_kv_lora, cfg.dsa_v_head
        Hi, Di, topk = cfg.dsa_index_heads, cfg.dsa_index_dim, cfg.dsa_topk
        T, eps = x.shape[0], cfg.rms_norm_eps
        cos, sin = ops.rope_cos_sin(ctx["positions"], rope, cfg.rope_theta, None)
        ql = ops.rmsnorm(ops.linear(x, p[pre + "mla_q_down"]), p[pre + "mla_q_norm"], eps)
        q = ops.linear(ql, p[pre + "mla_q_up"]).view(T, H, nope + rope)
        q_rope = ops.apply_rope(q[..., nope:].contiguous(), cos, sin)
        kvd = ops.linear(x, p[pre + "mla_kv_down"])
        c = ops.rmsnorm(kvd[:, :kvl].contiguous(), p[pre + "mla_kv_norm"], eps)
        k_rope = ops.apply_rope(kvd[:, None, kvl:].contiguous(), cos, sin)[:, 0]
        w = p[pre + "mla_kv_up"].view(H, nope + vh, kvl)
        w_uk, w_uv = w[:, :nope], w[:, nope:]
        qf = torch.cat([torch.einsum("thn,hnc->thc", q[..., :nope].float(), w_uk.float()).to(x.dtype), q_rope], -1)
        kv_new = torch.cat([c, k_rope], -1)
        scale = (nope + rope) ** -0.5
        if topk > 0:
            qi = ops.linear(x, p[pre + "idx_wq"]).view(T, Hi, Di)
            ki = ops.linear(x, p[pre + "idx_wk"])
            hw = ops.linear(x, p[pre + "idx_w"]) * Hi ** -0.5
        if ctx["mode"] == "prefill":
            starts, ends = D.causal_ranges(ctx["cu_t"], T)
            if topk > 0:
                idx = D.topk_indices(D.indexer_logits(qi, ki, hw, starts, ends), topk)
                lat, _ = D.sparse_mla_attention(qf, kv_new, idx, kvl, scale)
            else:
                lat, _ = D.dense_mla_attention(qf, kv_new, starts, ends, kvl, scale)
            fin = []
            for j, (a, b) in enumerate(zip(ctx["cu"], ctx["cu"][1:])):
                buf = kv_new.new_zeros(ctx["cap"][j], kv_new.shape[1])
                buf[: b - a] = kv_new[a:b]
                kb = None
                if topk > 0:
                    kb = ki.new_zeros(ctx["cap"][j], Di)
                    kb[: b - a] = ki[a:b]
                fin.append([buf, kb])
            ctx["out"][i] = fin
        else:
            cache, lens = ctx["cache"][i], ctx["lens"]
            for j in range(T):
                cache[j][0][lens[j]] = kv_new[j]
                if topk > 0:
                    cache[j][1][lens[j]] = ki[j]
            Lmax = max(lens) + 1
            n = torch.tensor([l_ + 1 for l_ in lens], device=x.device)
            cut = lambda t: F.pad(t[:Lmax], (0, 0, 0, max(0, Lmax - t.shape[0])))          # short requests own short buffers
            KV = torch.stack([cut(cb[0]) for cb in cache]).float()                          # [B, Lmax, C]
            beyond = torch.arange(Lmax, device=x.device)[None, :] >= n[:, None]             # [B, Lmax]
            sc = torch.einsum("bhc,blc->bhl", qf.float(), KV) * scale
            sc = sc.masked_fill(beyond[:, None, :], float("-inf"))
            if topk > 0:
                KI = torch.stack([cut(cb[1]) for cb in cache]).float()
                il = (F.relu(torch.einsum("bhd,bld->bhl", qi.float(), KI)) * hw.float()[..., None]).sum(1)
                il = il.masked_fill(beyond, float("-inf"))
                k_ = min(topk, Lmax)
                val, sel = il.sort(dim=-1, descending=True, stable=True)         # ties: the earlier position, as in training
                val, sel = val[:, :k_], sel[:, :k_]
                keep = torch.zeros_like(beyond).scatter_(1, sel, torch.isfinite(val))
                sc = sc.masked_fill(~keep[:, None, :], float("-inf"))
            lat = torch.einsum("bhl,blc->bhc", torch.softmax(sc, -1), KV[..., :kvl]).to(x.dtype)
        o = torch.einsum("thc,hvc->thv", lat.float(), w_uv.float()).to(x.dtype).reshape(T, H * vh)
        return ops.linear(o, p[pre + "mla_o"])

    def _layer(self, i, h, x, cos, sin, attn, tp, next_norm, cache):
        """One decoder layer.  ``h`` is the residual stream, ``x`` its normed copy (input of the attention
        block); returns the new ``(h, x)`` where ``x`` is already normed with ``next_norm`` (the next layer's
        input norm or the final norm), so every residual add is fused with the norm that follows it."""
        cfg, p = self.cfg, self.p
        pre = f"layers.{i}."
        if (pre + "gdn_qkvz") in p or (pre + "mla_q_down") in p:
            a = self._gdn(i, x) if (pre + "gdn_qkvz") in p else self._mla(i, x)
            x, h = ops.add_rmsnorm(a, h, p[pre + "post_norm"], cfg.rms_norm_eps)
            m, _ = self._mlp(i, x, tp)
            x, h = ops.add_rmsnorm(m, h, next_norm, cfg.rms_norm_eps)
            return h, x
        hd = cfg.head_dim
        nq, nkv = cfg.num_attention_heads // self.tp_size, cfg.num_query_groups // self.tp_size
        qkv = ops.linear(x, p[pre + "qkv"], p.get(pre + "qkv_bias"))
        if self.lora:
            qkv = self._lora_add(pre + "qkv", x, qkv)
        T = qkv.shape[0]
        kc, vc, slots, dense = cache
        q, k, v = ops.qkv_post(qkv, nq, nkv, p.get(pre + "q_norm") if cfg.qk_layernorm else None,
                               p.get(pre + "k_norm") if cfg.qk_layernorm else None, cos, sin, cfg.rms_norm_eps,
                               kc[i], vc[i], slots, dense)
        o = attn(i, q, k, v).reshape(T, nq * hd)
        if cfg.attention_output_gate:      # Qwen3.5: the attention output is gated per feature by a sigmoid of a projection of x
            o = o * torch.sigmoid(ops.linear(x, p[pre + "attn_gate"]).float()).to(o.dtype)
        if cfg.sandwich_norm:
            # h += norm(attention(norm(h))); h += norm(mlp(norm(h))): the extra norms sit between the reduction and the add
            a = ops.linear(o, p[pre + "o"])
            if self.lora:
                a = self._lora_add(pre + "o", o, a)
            a = ops.rmsnorm(self._allreduce(a, tp), p[pre + "post_attn_norm"], cfg.rms_norm_eps)
            x, h = ops.add_rmsnorm(a, h, p[pre + "post_norm"], cfg.rms_norm_eps)
            m, reduce_over = self._mlp(i, x, tp)
            if reduce_over is not None:
                m = self._allreduce(m, reduce_over)
            m = ops.rmsnorm(m, p[pre + "post_mlp_norm"], cfg.rms_norm_eps)
            x, h = ops.add_rmsnorm(m, h, next_norm, cfg.rms_norm_eps)
            return h, x
        comm = self._fused(tp, T, cfg.hidden_size) if not self.lora else None     # adapters add to the partial sums: plain path
        if comm is not None:
            h, x = comm.gemm_ar_add_rmsnorm(o, p[pre + "o"], h, p[pre + "post_norm"], cfg.rms_norm_eps)
        else:
            a = ops.linear(o, p[pre + "o"])
            if self.lora:
                a = self._lora_add(pre + "o", o, a)
            a = self._allreduce(a, tp)
            x, h = ops.add_rmsnorm(a, h, p[pre + "post_norm"], cfg.rms_norm_eps)
        if comm is not None and (pre + "router") not in p:
            a = ops.linear_swiglu(x, p[pre + "gate_up"])
            return comm.gemm_ar_add_rmsnorm(a, p[pre + "down"], h, next_norm, cfg.rms_norm_eps)
        m, reduce_over = self._mlp(i, x, tp)
        if reduce_over is not None:       # partial sums: over TP ranks (dense MLP) or over EP ranks (each holds some experts)
            m = self._allreduce(m, reduce_over)
        x, h = ops.add_rmsnorm(m, h, next_norm, cfg.rms_norm_eps)
        return h, x

    def _run(self, tokens, positions, attn, tp, cache, image=None, prenorm: bool = False):
        """The trunk.  Returns the final-norm output of every row; with ``prenorm`` also the residual stream before the
        final norm (the input of the multi-token-prediction block)."""
        cfg, p = self.cfg, self.p
        h = self._embed(tokens, tp)
        if image is not None:      # (rows, embeddings): image placeholder rows take the vision tower's output
            h = h.index_copy(0, image[0], image[1].to(h.dtype))
        cos, sin = ops.rope_cos_sin(positions, cfg.rotary_dim, cfg.rope_theta, cfg.mrope_section)
        x = ops.rmsnorm(h, p["layers.0.input_norm"], cfg.rms_norm_eps)
        for i in range(cfg.num_layers):
            nxt = p[f"layers.{i + 1}.input_norm"] if i + 1 < cfg.num_layers else p["final_norm"]
            h, x = self._layer(i, h, x, cos, sin, attn, tp, nxt, cache)
        return (x, h) if prenorm else x

    # ------------------------------------------------------------------ entry points
    def forward_prefill(self, tokens, positions, cu_seqlens, slots, kv, last_rows, tp: GroupInfo, max_seqlen=None,
                        image=None, return_hidden: bool = False):
        def attn(i, q, k, v):
            return ops.attention_varlen(q, k, v, cu_seqlens, causal=True, max_seqlen=max_seqlen)

        if return_hidden:      # speculative decoding: the draft block reads the trunk's pre-norm hidden of every row
            x, h = self._run(tokens, positions, attn, tp, (kv[:, 0], kv[:, 1], slots, True), image=image, prenorm=True)
            return self._logits(x[last_rows], tp), h
        h = self._run(tokens, positions, attn, tp, (kv[:, 0], kv[:, 1], slots, True), image=image)
        return self._logits(h[last_rows], tp)

    # ------------------------------------------------------------------ speculative decoding (draft = the MTP block)
    def forward_rows(self, tokens, positions, block_tables, context_lens, slots, kv, tp: GroupInfo):
        """A decode-shaped pass in which a request may own SEVERAL rows (its newest token and draft tokens after it):
        row ``j`` writes its K/V to ``slots[j]`` and attends to the first ``context_lens[j]`` positions of its block
        table, which include the rows of the same request before it - every layer writes all rows' K/V before its
        attention runs.  Returns ``(logits, pre-norm hidden)`` per row."""
        def attn(i, q, k, v):
            return ops.paged_decode_attention(q, kv[i, 0], kv[i, 1], block_tables, context_lens)

        x, h = self._run(tokens, positions, attn, tp, (kv[:, 0], kv[:, 1], slots, False), prenorm=True)
        return self._logits(x, tp), h

    def _mtp_block(self, h_prev, next_tokens, positions, attn, tp, cache):
        """The multi-token-prediction block on rows: ``h_prev`` is the trunk's pre-norm hidden at a position,
        ``next_tokens`` the token that FOLLOWS that position; the output predicts the token after that one
        (relax_b200/models/mtp.py MTPBlock.forward: concat of the two normed inputs, projection, one decoder layer,
        final norm, the shared LM head)."""
        cfg, p = self.cfg, self.p
        L = cfg.num_layers
        eps = cfg.rms_norm_eps
        emb = self._embed(next_tokens, tp)
        x = torch.cat([ops.rmsnorm(emb, p["mtp.enorm"], eps), ops.rmsnorm(h_prev.to(emb.dtype), p["mtp.hnorm"], eps)], -1)
        h = ops.linear(x, p["mtp.eh_proj"])
        cos, sin = ops.rope_cos_sin(positions, cfg.rotary_dim, cfg.rope_theta, cfg.mrope_section)
        xin = ops.rmsnorm(h, p[f"layers.{L}.input_norm"], eps)
        h_out, xn = self._layer(L, h, xin, cos, sin, attn, tp, p["mtp.final_norm"], cache)
        return xn, h_out         # h_out: the block's own un-normalised output (stands in for the trunk's hidden when proposals are chained)

    def forward_mtp_rows(self, h_prev, next_tokens, positions, block_tables, context_lens, slots, kv, tp: GroupInfo, out_rows=None,
                         return_hidden: bool = False):
        """Draft logits from decode-shaped rows (layer ``num_layers`` of ``kv`` is the block's own cache); with
        ``return_hidden`` also the block's output hidden of the same rows."""
        L = self.cfg.num_layers

        def attn(i, q, k, v):
            return ops.paged_decode_attention(q, kv[L, 0], kv[L, 1], block_tables, context_lens)

        xn, ho = self._mtp_block(h_prev, next_tokens, positions, attn, tp, (kv[:, 0], kv[:, 1], slots, False))
        if out_rows is not None:
            xn, ho = xn[out_rows], ho[out_rows]
        return (self._logits(xn, tp), ho) if return_hidden else self._logits(xn, tp)

    def forward_mtp_prefill(self, h_prev, next_tokens, positions, cu_seqlens, slots, kv, last_rows, tp: GroupInfo, max_seqlen=None):
        """The block over whole prompts (fills its cache for every prompt position); draft logits and the block's
        output hidden of the last rows."""
        def attn(i, q, k, v):
            return ops.attention_varlen(q, k, v, cu_seqlens, causal=True, max_seqlen=max_seqlen)

        xn, ho = self._mtp_block(h_prev, next_tokens, positions, attn, tp, (kv[:, 0], kv[:, 1], slots, True))
        return self._logits(xn[last_rows], tp), ho[last_rows]

    def forward_decode(self, tokens, positions, block_tables, context_lens, slots, kv, tp: GroupInfo):
        def attn(i, q, k, v):
            return ops.paged_decode_attention(q, kv[i, 0], kv[i, 1], block_tables, context_lens)

        h = self._run(tokens, positions, attn, tp, (kv[:, 0], kv[:, 1], slots, False))
        return self._logits(h, tp)
