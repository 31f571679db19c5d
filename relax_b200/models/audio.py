"""Audio tower and the omni wrapper: log-mel features -> two stride-2 convolutions -> non-causal transformer blocks
over each clip -> pairs of frames merged and projected into the language model's embedding space; text, image and
audio embeddings are merged at their placeholder tokens.

Covers the audio side of the reference's Qwen3-Omni thinker (relax/models/qwen_omni/modeling_qwen3_omni/: model.py,
utils.py placeholders and position index) on this framework's packed layout: all clips of a micro-batch are
concatenated along time with ``cu_seqlens`` boundaries, the attention kernel is the same varlen flash attention
(non-causal) the vision tower uses, and the number of output tokens per clip equals
:func:`relax_b200.data.multimodal.audio_token_count`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .vision import merge_image_embeddings


@dataclass
class AudioConfig:
    n_mels: int = 128
    hidden_size: int = 1280
    num_heads: int = 20
    intermediate_size: int = 5120
    depth: int = 32
    out_hidden_size: int = 2048
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads


def sinusoid_positions(n: int, dim: int, device=None) -> torch.Tensor:
    half = dim // 2
    inv = torch.exp(-math.log(10000.0) * torch.arange(half, device=device, dtype=torch.float32) / max(1, half - 1))
    ang = torch.arange(n, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([ang.sin(), ang.cos()], -1)


class AudioBlock(nn.Module):
    def __init__(self, cfg: AudioConfig, dtype, device, gen):
        super().__init__()
        self.cfg = cfg
        h, f = cfg.hidden_size, cfg.intermediate_size
        mk = lambda *s, std=0.02: nn.Parameter((torch.randn(*s, generator=gen) * std).to(device=device, dtype=dtype))
        zeros = lambda n: nn.Parameter(torch.zeros(n, dtype=dtype, device=device))
        ones = lambda n: nn.Parameter(torch.ones(n, dtype=dtype, device=device))
        self.ln1_w, self.ln1_b, self.ln2_w, self.ln2_b = ones(h), zeros(h), ones(h), zeros(h)
        self.qkv, self.qkv_bias = mk(3 * h, h), zeros(3 * h)
        self.proj, self.proj_bias = mk(h, h, std=0.02 / math.sqrt(2 * cfg.depth)), zeros(h)
        self.fc1, self.fc1_bias = mk(f, h), zeros(f)
        self.fc2, self.fc2_bias = mk(h, f, std=0.02 / math.sqrt(2 * cfg.depth)), zeros(h)

    def forward(self, x, cu_seqlens, max_seqlen):
        cfg = self.cfg
        y = F.layer_norm(x.float(), (cfg.hidden_size,), self.ln1_w.float(), self.ln1_b.float(), cfg.eps).to(x.dtype)
        qkv = ops.linear(y, self.qkv, self.qkv_bias).view(-1, 3, cfg.num_heads, cfg.head_dim)
        o = ops.attention_varlen(qkv[:, 0].contiguous(), qkv[:, 1].contiguous(), qkv[:, 2].contiguous(), cu_seqlens,
                                 causal=False, max_seqlen=max_seqlen)
        x = x + ops.linear(o.reshape(o.shape[0], -1), self.proj, self.proj_bias)
        y = F.layer_norm(x.float(), (cfg.hidden_size,), self.ln2_w.float(), self.ln2_b.float(), cfg.eps).to(x.dtype)
        return x + ops.linear(F.gelu(ops.linear(y, self.fc1, self.fc1_bias)), self.fc2, self.fc2_bias)


class AudioEncoder(nn.Module):
    def __init__(self, cfg: AudioConfig, dtype=torch.float32, device="cpu", seed: int = 0):
        super().__init__()
        self.cfg = cfg
        gen = torch.Generator(device="cpu").manual_seed(seed)
        h = cfg.hidden_size
        mk = lambda *s, std=0.02: nn.Parameter((torch.randn(*s, generator=gen) * std).to(device=device, dtype=dtype))
        self.conv1_w, self.conv1_b = mk(h, cfg.n_mels, 3), nn.Parameter(torch.zeros(h, dtype=dtype, device=device))
        self.conv2_w, self.conv2_b = mk(h, h, 3), nn.Parameter(torch.zeros(h, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([AudioBlock(cfg, dtype, device, gen) for _ in range(cfg.depth)])
        self.ln_post_w = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        self.ln_post_b = nn.Parameter(torch.zeros(h, dtype=dtype, device=device))
        self.merge_fc1 = mk(h, 2 * h)
        self.merge_fc2 = mk(cfg.out_hidden_size, h)

    def _stem(self, mel: torch.Tensor) -> torch.Tensor:
        """``[n_mels, frames]`` -> ``[frames', hidden]``: conv (stride 1) + GELU, conv (stride 2) + GELU, positions."""
        x = mel.to(self.conv1_w.dtype)[None]
        x = F.gelu(F.conv1d(x, self.conv1_w, self.conv1_b, stride=1, padding=1))
        x = F.gelu(F.conv1d(x, self.conv2_w, self.conv2_b, stride=2, padding=1))[0].t()
        return x + sinusoid_positions(x.shape[0], x.shape[1], x.device).to(x.dtype)

    def forward(self, mels: Sequence[torch.Tensor]):
        """``mels``: one ``[n_mels, frames]`` tensor per clip.  Returns ``(embeddings [sum tokens, out_hidden],
        tokens per clip)``."""
        seqs = [self._stem(m) for m in mels]
        lens = [s.shape[0] - s.shape[0] % 2 if s.shape[0] >= 2 else s.shape[0] for s in seqs]
        seqs = [s[:n] for s, n in zip(seqs, lens)]
        x = torch.cat(seqs)
        cu = torch.zeros(len(seqs) + 1, dtype=torch.int32, device=x.device)
        cu[1:] = torch.tensor(lens, device=x.device).cumsum(0)
        for blk in self.blocks:
            x = blk(x, cu, max(lens))
        x = F.layer_norm(x.float(), (self.cfg.hidden_size,), self.ln_post_w.float(), self.ln_post_b.float(), self.cfg.eps).to(x.dtype)
        outs, counts, o = [], [], 0
        for n in lens:
            seg = x[o:o + n]
            o += n
            if n >= 2:
                seg = seg.reshape(n // 2, 2 * self.cfg.hidden_size)
            else:
                seg = torch.cat([seg, seg], -1)
            outs.append(seg)
            counts.append(seg.shape[0])
        y = torch.cat(outs)
        return ops.linear(F.gelu(ops.linear(y, self.merge_fc1)), self.merge_fc2), counts


class OmniModel(nn.Module):
    """Language model + optional vision and audio towers; embeddings of each modality replace that modality's
    placeholder tokens in order of appearance."""

    def __init__(self, lm, vision=None, audio: Optional[AudioEncoder] = None, image_token_id: int = -1, audio_token_id: int = -2):
        super().__init__()
        self.lm, self.vision, self.audio = lm, vision, audio
        self.image_token_id, self.audio_token_id = image_token_id, audio_token_id

    def forward(self, tokens, positions, cu_seqlens, pixel_patches=None, grid_thw=None, audio_mels=None, max_seqlen=None):
        emb = self.lm.embedding.word_embeddings(tokens, False)
        if pixel_patches is not None and pixel_patches.numel():
            emb = merge_image_embeddings(emb, self.vision(pixel_patches, grid_thw), tokens, self.image_token_id)
        if audio_mels:
            a, _ = self.audio(audio_mels)
            emb = merge_image_embeddings(emb, a, tokens, self.audio_token_id)
        return self.lm(tokens, positions, cu_seqlens, inputs_embeds=emb, max_seqlen=max_seqlen)
