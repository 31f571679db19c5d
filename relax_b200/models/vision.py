"""Vision encoder and multimodal glue for the VL model families (Qwen2.5-VL style; the reference trains them
through Megatron-Bridge models and ships its own ViT for DotsOCR, relax/models/dots_ocr/vision.py:58-217, and the
M-RoPE index of Qwen3-Omni, relax/models/qwen_omni/modeling_qwen3_omni/utils.py:57).

* :class:`VisionEncoder` - patch embedding over flattened ``[C x Tp x P x P]`` patches, 2-D rotary position
  embedding (row / column halves), pre-norm blocks with full (non-causal) variable-length attention per image -
  the same flash-attention kernel as the language model, ``causal=False`` - and SwiGLU MLPs, then a patch merger
  that folds ``merge x merge`` neighbouring patches into one language-model token.
* :func:`mrope_positions` - the three position streams (temporal, height, width) of multimodal RoPE: text tokens
  advance all three together; the tokens of an image share one temporal index and carry their grid row / column;
  the text after an image continues from the largest index used so far.
* :class:`VLModel` - language model + encoder: image tokens in the prompt are replaced by encoder outputs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn as nn

from .. import ops


@dataclass
class VisionConfig:
    patch_size: int = 14
    temporal_patch_size: int = 2
    in_channels: int = 3
    hidden_size: int = 1280
    num_heads: int = 16
    intermediate_size: int = 3420
    depth: int = 32
    spatial_merge_size: int = 2
    out_hidden_size: int = 3584
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    patch_norm: bool = False          # RMSNorm on the patch embeddings (dots.ocr)
    post_trunk_norm: bool = False     # RMSNorm after the last block (dots.ocr)
    merger_layernorm: bool = False    # LayerNorm with bias in front of the merger instead of RMSNorm (dots.ocr)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


def vision_rope_tables(grid_thw: torch.Tensor, head_dim: int, theta: float, merge: int):
    """cos/sin ``[N, head_dim/2]`` for all patches of all images, in the merge-window-major order the patches are
    fed in (``merge x merge`` neighbours adjacent): first half of the frequencies follows the row, second the column."""
    quarter = head_dim // 4
    inv = 1.0 / (theta ** (torch.arange(0, quarter, dtype=torch.float32, device=grid_thw.device) / quarter))
    rows, cols = [], []
    for t, h, w in grid_thw.tolist():
        r = torch.arange(h, device=grid_thw.device).view(h // merge, merge, 1, 1).expand(h // merge, merge, w // merge, merge)
        c = torch.arange(w, device=grid_thw.device).view(1, 1, w // merge, merge).expand(h // merge, merge, w // merge, merge)
        r = r.permute(0, 2, 1, 3).reshape(-1)
        c = c.permute(0, 2, 1, 3).reshape(-1)
        rows.append(r.repeat(t))
        cols.append(c.repeat(t))
    r, c = torch.cat(rows).float(), torch.cat(cols).float()
    ang = torch.cat([r[:, None] * inv[None, :], c[:, None] * inv[None, :]], -1)
    return ang.cos(), ang.sin()


class VisionBlock(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype, device, gen):
        super().__init__()
        h, f = cfg.hidden_size, cfg.intermediate_size
        self.cfg = cfg
        mk = lambda *s, std=0.02: nn.Parameter((torch.randn(*s, generator=gen) * std).to(device=device, dtype=dtype))
        self.norm1 = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        self.norm2 = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        self.qkv = mk(3 * h, h)
        self.qkv_bias = nn.Parameter(torch.zeros(3 * h, dtype=dtype, device=device))
        self.proj = mk(h, h, std=0.02 / math.sqrt(2 * cfg.depth))
        # The MLP width is padded to a multiple of 64 with zero rows (fc1) / zero columns (fc2): 3420 (Qwen2.5-VL)
        # becomes 3456, every row stride is a multiple of 16 bytes (what the TMA-fed GEMMs and the vectorised
        # activation kernel need) and the function is unchanged - silu(0) * 0 = 0 and the padding receives zero
        # gradients, so it stays zero through training.
        fp = (f + 63) // 64 * 64
        self.f, self.f_pad = f, fp
        fc1, fc2 = mk(2 * f, h), mk(h, f, std=0.02 / math.sqrt(2 * cfg.depth))
        if fp != f:
            w1 = torch.zeros(2 * fp, h, dtype=dtype, device=device)
            w1[:f], w1[fp:fp + f] = fc1.data[:f], fc1.data[f:]
            w2 = torch.zeros(h, fp, dtype=dtype, device=device)
            w2[:, :f] = fc2.data
            fc1, fc2 = nn.Parameter(w1), nn.Parameter(w2)
        self.fc1 = fc1                 # [gate; up], each f_pad rows
        self.fc2 = fc2
        # Qwen2.5-VL's tower has a bias on every linear (zero here until a checkpoint is loaded)
        zb = lambda n: nn.Parameter(torch.zeros(n, dtype=dtype, device=device))
        self.proj_bias, self.fc1_bias, self.fc2_bias = zb(h), zb(2 * fp), zb(h)

    def forward(self, x, cos, sin, cu_seqlens, max_seqlen):
        cfg = self.cfg
        n, hd = cfg.num_heads, cfg.head_dim
        y = ops.rmsnorm(x, self.norm1, cfg.rms_norm_eps)
        qkv = ops.linear(y, self.qkv, self.qkv_bias).view(-1, 3, n, hd)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        q, k = ops.apply_rope(q.contiguous(), cos, sin), ops.apply_rope(k.contiguous(), cos, sin)
        o = ops.attention_varlen(q, k, v.contiguous(), cu_seqlens, causal=False, max_seqlen=max_seqlen)
        # the biases are added as separate elementwise steps: these linears then take exactly the bias-free GEMM paths
        # (the tower is a small share of a step; the q/k/v bias above rides in the GEMM epilogue)
        x = x + (ops.linear(o.reshape(o.shape[0], -1), self.proj) + self.proj_bias)
        y = ops.rmsnorm(x, self.norm2, cfg.rms_norm_eps)
        return x + (ops.linear(ops.swiglu(ops.linear(y, self.fc1) + self.fc1_bias), self.fc2) + self.fc2_bias)


class VisionEncoder(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype=torch.float32, device="cpu", seed: int = 0):
        super().__init__()
        self.cfg = cfg
        gen = torch.Generator(device="cpu").manual_seed(seed)
        h = cfg.hidden_size
        self.patch_embed = nn.Parameter((torch.randn(h, cfg.patch_dim, generator=gen) * 0.02).to(device=device, dtype=dtype))
        self.blocks = nn.ModuleList([VisionBlock(cfg, dtype, device, gen) for _ in range(cfg.depth)])
        m2 = cfg.spatial_merge_size ** 2
        self.merger_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        if cfg.patch_norm:
            self.patch_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        if cfg.post_trunk_norm:
            self.post_trunk_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        if cfg.merger_layernorm:
            self.merger_norm_bias = nn.Parameter(torch.zeros(h, dtype=dtype, device=device))
        self.merger_fc1 = nn.Parameter((torch.randn(h * m2, h * m2, generator=gen) * 0.02).to(device=device, dtype=dtype))
        self.merger_fc2 = nn.Parameter((torch.randn(cfg.out_hidden_size, h * m2, generator=gen) * 0.02).to(device=device, dtype=dtype))
        self.merger_fc1_bias = nn.Parameter(torch.zeros(h * m2, dtype=dtype, device=device))
        self.merger_fc2_bias = nn.Parameter(torch.zeros(cfg.out_hidden_size, dtype=dtype, device=device))

    def forward(self, pixel_patches: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """``pixel_patches [N, patch_dim]`` (all images concatenated, merge-window-major), ``grid_thw [n_img, 3]`` in
        patches.  Returns ``[N / merge^2, out_hidden]`` language-model embeddings."""
        cfg = self.cfg
        x = ops.linear(pixel_patches.to(self.patch_embed.dtype), self.patch_embed)
        if cfg.patch_norm:
            x = ops.rmsnorm(x, self.patch_norm, cfg.rms_norm_eps)
        cos, sin = vision_rope_tables(grid_thw, cfg.head_dim, cfg.rope_theta, cfg.spatial_merge_size)
        lens = (grid_thw[:, 0] * grid_thw[:, 1] * grid_thw[:, 2]).to(torch.int32)
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32, device=x.device)
        cu[1:] = lens.cumsum(0)
        mx = int(lens.max())
        for blk in self.blocks:
            x = blk(x, cos, sin, cu, mx)
        if cfg.post_trunk_norm:
            x = ops.rmsnorm(x, self.post_trunk_norm, cfg.rms_norm_eps)
        if cfg.merger_layernorm:
            x = torch.nn.functional.layer_norm(x.float(), (cfg.hidden_size,), self.merger_norm.float(), self.merger_norm_bias.float(),
                                               1e-6).to(x.dtype)
        else:
            x = ops.rmsnorm(x, self.merger_norm, cfg.rms_norm_eps)
        x = x.view(-1, cfg.hidden_size * cfg.spatial_merge_size ** 2)
        return ops.linear(torch.nn.functional.gelu(ops.linear(x, self.merger_fc1) + self.merger_fc1_bias), self.merger_fc2) \
            + self.merger_fc2_bias


def mrope_positions(input_ids: Sequence[int], image_grid_thw: Sequence[Sequence[int]], image_token_id: int,
                    spatial_merge_size: int = 2, device="cpu") -> torch.Tensor:
    """``[3, T]`` (temporal, height, width) position ids of one sequence whose image placeholders are runs of
    ``image_token_id`` (one run per image, ``t * h/merge * w/merge`` tokens long)."""
    ids = list(input_ids)
    T = len(ids)
    pos = torch.zeros(3, T, dtype=torch.long)
    nxt, i, img = 0, 0, 0
    while i < T:
        if ids[i] != image_token_id:
            pos[:, i] = nxt
            nxt += 1
            i += 1
            continue
        if img >= len(image_grid_thw):
            raise ValueError(f"placeholder tokens at position {i} but only {len(image_grid_thw)} image grid(s) given")
        t, h, w = image_grid_thw[img]
        gh, gw = h // spatial_merge_size, w // spatial_merge_size
        n = t * gh * gw
        if ids[i:i + n] != [image_token_id] * n:
            raise ValueError(f"image {img}: expected a run of {n} placeholder tokens at position {i}")
        tt = torch.arange(t).view(t, 1, 1).expand(t, gh, gw).reshape(-1)
        hh = torch.arange(gh).view(1, gh, 1).expand(t, gh, gw).reshape(-1)
        ww = torch.arange(gw).view(1, 1, gw).expand(t, gh, gw).reshape(-1)
        pos[0, i:i + n], pos[1, i:i + n], pos[2, i:i + n] = nxt + tt, nxt + hh, nxt + ww
        nxt = nxt + max(t, gh, gw)
        i += n
        img += 1
    if img != len(image_grid_thw):
        raise ValueError(f"{len(image_grid_thw)} images given, {img} placeholder runs found")
    return pos.to(device)


def merge_image_embeddings(text_embeds: torch.Tensor, image_embeds: torch.Tensor, input_ids: torch.Tensor,
                           image_token_id: int) -> torch.Tensor:
    mask = input_ids == image_token_id
    if int(mask.sum()) != image_embeds.shape[0]:
        raise ValueError(f"{int(mask.sum())} image tokens in the prompt but {image_embeds.shape[0]} image embeddings")
    out = text_embeds.clone()
    out[mask] = image_embeds.to(out.dtype)
    return out


def vision_config_from_model(mc) -> VisionConfig:
    """The encoder configuration of a VL preset (``ModelConfig.vision`` of models/config.py)."""
    v = mc.vision
    return VisionConfig(patch_size=v.patch_size, temporal_patch_size=v.temporal_patch_size, in_channels=v.in_channels,
                        hidden_size=v.hidden_size, num_heads=v.num_heads, intermediate_size=v.ffn_hidden_size,
                        depth=v.num_layers, spatial_merge_size=v.spatial_merge_size, out_hidden_size=v.out_hidden_size,
                        rms_norm_eps=v.rms_norm_eps if v.rms_norm_eps is not None else mc.rms_norm_eps,
                        patch_norm=v.patch_norm, post_trunk_norm=v.post_trunk_norm, merger_layernorm=v.merger_layernorm)


class VLModel(nn.Module):
    """Language model + vision encoder.  ``forward`` returns the final hidden states like ``GPTModel.forward``."""

    def __init__(self, lm, vision: VisionEncoder, image_token_id: int, branch_sync=None):
        super().__init__()
        self.lm, self.vision, self.image_token_id = lm, vision, image_token_id
        # a parallel.collective_utils.ConditionalBranchSync over the data-parallel group: when only some ranks
        # have images in a micro-batch the others run the tower on one placeholder window (times zero), so the
        # gradient reduction sees the vision parameters on every rank
        self.branch_sync = branch_sync

    def _dummy_vision(self):
        m = self.vision.cfg.spatial_merge_size
        p = torch.zeros(m * m, self.vision.cfg.patch_dim, dtype=self.vision.patch_embed.dtype, device=self.vision.patch_embed.device)
        return self.vision(p, torch.tensor([[1, m, m]], device=p.device)).sum()

    def forward(self, tokens, positions, cu_seqlens, pixel_patches=None, grid_thw=None, max_seqlen=None):
        emb = self.lm.embedding.word_embeddings(tokens, False)
        has = pixel_patches is not None and pixel_patches.numel() > 0
        if self.branch_sync is not None and torch.is_grad_enabled():
            r = self.branch_sync.run(has, lambda: self.vision(pixel_patches, grid_thw), self._dummy_vision)
            if has:
                emb = merge_image_embeddings(emb, r, tokens, self.image_token_id)
            elif r is not None:
                emb = emb + r.to(emb.dtype)
        elif has:
            emb = merge_image_embeddings(emb, self.vision(pixel_patches, grid_thw), tokens, self.image_token_id)
        return self.lm(tokens, positions, cu_seqlens, inputs_embeds=emb, max_seqlen=max_seqlen)


# ----------------------------------------------------------------------------- Hugging Face names of the tower
def vision_state_to_hf(enc: "VisionEncoder", prefix: str = "visual.") -> dict:
    """This tower's parameters under the names of a Qwen2.5-VL checkpoint (``visual.patch_embed.proj.weight`` as the
    3-D convolution kernel, ``visual.blocks.N.attn.qkv / proj``, ``mlp.gate_proj / up_proj / down_proj`` with the width
    padding removed, ``visual.merger.ln_q / mlp.0 / mlp.2``)."""
    c = enc.cfg
    out = {prefix + "patch_embed.proj.weight": enc.patch_embed.detach().view(c.hidden_size, c.in_channels, c.temporal_patch_size,
                                                                             c.patch_size, c.patch_size)}
    for i, b in enumerate(enc.blocks):
        p, f, fp = f"{prefix}blocks.{i}.", b.f, b.f_pad
        out[p + "norm1.weight"], out[p + "norm2.weight"] = b.norm1.detach(), b.norm2.detach()
        out[p + "attn.qkv.weight"], out[p + "attn.qkv.bias"] = b.qkv.detach(), b.qkv_bias.detach()
        out[p + "attn.proj.weight"], out[p + "attn.proj.bias"] = b.proj.detach(), b.proj_bias.detach()
        out[p + "mlp.gate_proj.weight"], out[p + "mlp.up_proj.weight"] = b.fc1.detach()[:f], b.fc1.detach()[fp:fp + f]
        out[p + "mlp.gate_proj.bias"], out[p + "mlp.up_proj.bias"] = b.fc1_bias.detach()[:f], b.fc1_bias.detach()[fp:fp + f]
        out[p + "mlp.down_proj.weight"], out[p + "mlp.down_proj.bias"] = b.fc2.detach()[:, :f], b.fc2_bias.detach()
    out[prefix + "merger.ln_q.weight"] = enc.merger_norm.detach()
    out[prefix + "merger.mlp.0.weight"], out[prefix + "merger.mlp.0.bias"] = enc.merger_fc1.detach(), enc.merger_fc1_bias.detach()
    out[prefix + "merger.mlp.2.weight"], out[prefix + "merger.mlp.2.bias"] = enc.merger_fc2.detach(), enc.merger_fc2_bias.detach()
    return {k: v.contiguous() for k, v in out.items()}


@torch.no_grad()
def load_vision_from_hf(enc: "VisionEncoder", hf: dict, strict: bool = True) -> list:
    """Fill the tower from a Hugging Face state dict; the prefix may be ``visual.`` or ``model.visual.`` (newer
    checkpoints).  Returns the tower tensors for which the checkpoint had nothing (empty when ``strict``)."""
    prefix = next((p for p in ("model.visual.", "visual.") if any(k.startswith(p) for k in hf)), None)
    if prefix is None:
        if strict:
            raise KeyError("the checkpoint holds no vision tower (no visual.* tensors)")
        return ["visual.*"]
    want = vision_state_to_hf(enc, prefix)
    missing = [k for k in want if k not in hf]
    if missing and strict:
        raise KeyError(f"vision tower tensors missing from the checkpoint: {missing[:4]} ...")
    g = lambda k: hf[prefix + k].to(enc.patch_embed.dtype)
    has = lambda k: (prefix + k) in hf
    if has("patch_embed.proj.weight"):
        enc.patch_embed.copy_(g("patch_embed.proj.weight").reshape(enc.patch_embed.shape))
    for i, b in enumerate(enc.blocks):
        p, f, fp = f"blocks.{i}.", b.f, b.f_pad
        for ours, theirs in ((b.norm1, "norm1.weight"), (b.norm2, "norm2.weight"), (b.qkv, "attn.qkv.weight"), (b.qkv_bias, "attn.qkv.bias"),
                             (b.proj, "attn.proj.weight"), (b.proj_bias, "attn.proj.bias"), (b.fc2_bias, "mlp.down_proj.bias")):
            if has(p + theirs):
                ours.copy_(g(p + theirs))
        if has(p + "mlp.gate_proj.weight"):
            b.fc1.zero_()
            b.fc1[:f], b.fc1[fp:fp + f] = g(p + "mlp.gate_proj.weight"), g(p + "mlp.up_proj.weight")
            b.fc2.zero_()
            b.fc2[:, :f] = g(p + "mlp.down_proj.weight")
        if has(p + "mlp.gate_proj.bias"):
            b.fc1_bias.zero_()
            b.fc1_bias[:f], b.fc1_bias[fp:fp + f] = g(p + "mlp.gate_proj.bias"), g(p + "mlp.up_proj.bias")
    for ours, theirs in ((enc.merger_norm, "merger.ln_q.weight"), (enc.merger_fc1, "merger.mlp.0.weight"), (enc.merger_fc1_bias, "merger.mlp.0.bias"),
                         (enc.merger_fc2, "merger.mlp.2.weight"), (enc.merger_fc2_bias, "merger.mlp.2.bias")):
        if has(theirs):
            ours.copy_(g(theirs))
    return missing
