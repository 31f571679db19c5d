"""Model shape descriptions and the named presets used by recipes and benchmarks.

The fields follow the MODEL_ARGS of the reference's ``scripts/models/*.sh``
(e.g. scripts/models/qwen3-8B.sh:4-18, scripts/models/qwen3-30B-A3B.sh:40-50).
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict, replace
from typing import Optional


@dataclass
class VisionConfig:
    num_layers: int = 32
    hidden_size: int = 1280
    num_heads: int = 16
    ffn_hidden_size: int = 3420
    patch_size: int = 14
    spatial_merge_size: int = 2
    in_channels: int = 3
    temporal_patch_size: int = 2
    out_hidden_size: int = 3584
    # dots.ocr's tower (relax/models/dots_ocr/vision.py): RMSNorm after the patch projection and after the last block, a
    # LayerNorm (with bias) in front of the merger, its own norm epsilon
    patch_norm: bool = False
    post_trunk_norm: bool = False
    merger_layernorm: bool = False
    rms_norm_eps: "float | None" = None


@dataclass
class ModelConfig:
    name: str = "tiny"
    num_layers: int = 2
    hidden_size: int = 256
    num_attention_heads: int = 4
    num_query_groups: int = 2
    head_dim: int = 64
    ffn_hidden_size: int = 688
    vocab_size: int = 1024
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    qk_layernorm: bool = True
    qkv_bias: bool = False
    tie_word_embeddings: bool = False
    # MoE
    num_experts: int = 0
    moe_top_k: int = 0
    moe_ffn_hidden_size: int = 0
    moe_router_norm_topk_prob: bool = True
    moe_aux_loss_coef: float = 0.0
    moe_layer_freq: int = 1
    moe_first_dense_layers: int = 0        # DeepSeek-V3 / GLM4-MoE: the first k layers keep a dense MLP
    moe_shared_expert_ffn: int = 0         # >0: an always-on shared expert of this width beside the routed ones
    moe_shared_expert_gate: bool = False   # Qwen2-MoE / Qwen3-Next: shared output scaled by sigmoid(gate(x))
    moe_router_score: str = "softmax"      # softmax | sigmoid (DeepSeek-V3 / GLM4-MoE)
    moe_router_bias: bool = False          # selection-only per-expert bias, balanced without an auxiliary loss
    moe_routed_scaling_factor: float = 1.0
    moe_router_bias_update_rate: float = 1e-3
    # multimodal
    vision: Optional[VisionConfig] = None
    mrope_section: Optional[tuple] = None  # (t, h, w) halves of head_dim/2
    image_token_id: int = -1
    # value / classification head
    value_head: bool = False
    num_classes: int = 0                  # >0: sequence-classification head on the last token
    # multi-token prediction blocks after the trunk (0 = none)
    mtp_num_layers: int = 0
    # Qwen3.5-style softmax attention: a sigmoid gate on the attention output (the query projection also produces one
    # gate value per query feature) and rotary embedding on the first `rotary_percent` of every head only
    attention_output_gate: bool = False
    rotary_percent: float = 1.0
    # GLM-4 dense: "sandwich" norms - the attention and MLP outputs are normalised once more before they join the residual
    sandwich_norm: bool = False
    # norm weights are stored zero-centred (gamma - 1) in this family's checkpoints (``--apply-layernorm-1p``); the model
    # keeps gamma, the Hugging Face conversion adds / removes the offset
    layernorm_zero_centered: bool = False
    # hybrid stacks: every `linear_attention_freq`-th layer is softmax attention, the others Gated DeltaNet (0 = all softmax)
    linear_attention_freq: int = 0
    gdn_k_heads: int = 2
    gdn_v_heads: int = 4
    gdn_head_dim: int = 32
    # multi-head latent attention (DeepSeek-V3 / GLM-4.7 style, dims below); with dsa_topk > 0 it is sparse (DSA)
    multi_latent_attention: bool = False
    dsa_topk: int = 0
    dsa_q_lora: int = 64
    dsa_kv_lora: int = 32
    dsa_nope: int = 16
    dsa_rope: int = 8
    dsa_v_head: int = 16
    dsa_index_heads: int = 4
    dsa_index_dim: int = 16
    dsa_indexer_loss_coef: float = 1.0
    dtype: str = "bf16"

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def is_moe_layer(self, layer_idx: int) -> bool:
        return self.is_moe and layer_idx >= self.moe_first_dense_layers and layer_idx % self.moe_layer_freq == 0

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_query_groups * self.head_dim

    @property
    def rotary_dim(self) -> int:
        """Leading features of a head that are rotated (even; the whole head unless ``rotary_percent`` < 1)."""
        return self.head_dim if self.rotary_percent >= 1.0 else max(2, int(self.head_dim * self.rotary_percent) // 2 * 2)

    def num_parameters(self) -> int:
        h, L = self.hidden_size, self.num_layers
        attn = h * (self.q_size * (2 if self.attention_output_gate else 1) + 2 * self.kv_size) + self.q_size * h
        if self.qk_layernorm:
            attn += 2 * self.head_dim
        if self.is_moe:
            mlp = self.num_experts * 3 * h * self.moe_ffn_hidden_size + h * self.num_experts
        else:
            mlp = 3 * h * self.ffn_hidden_size
        per_layer = attn + mlp + 2 * h
        emb = self.vocab_size * h
        out = 0 if self.tie_word_embeddings else self.vocab_size * h
        return L * per_layer + emb + out + h

    def to_dict(self):
        return asdict(self)


PRESETS: dict[str, ModelConfig] = {}


def _reg(c: ModelConfig):
    PRESETS[c.name] = c
    return c


# BASELINE config 0 ("tiny Qwen-style decoder")
_reg(ModelConfig(name="tiny", num_layers=2, hidden_size=256, num_attention_heads=4, num_query_groups=2,
                 head_dim=64, ffn_hidden_size=688, vocab_size=1024, dtype="fp32"))
_reg(ModelConfig(name="tiny-moe", num_layers=2, hidden_size=256, num_attention_heads=4, num_query_groups=2,
                 head_dim=64, ffn_hidden_size=688, vocab_size=1024, num_experts=8, moe_top_k=2,
                 moe_ffn_hidden_size=128, dtype="fp32"))
_reg(ModelConfig(name="tiny-next", num_layers=4, hidden_size=128, num_attention_heads=4, num_query_groups=2, head_dim=32,
                 ffn_hidden_size=256, vocab_size=512, linear_attention_freq=4, dtype="fp32"))
_reg(ModelConfig(name="tiny-vl", num_layers=2, hidden_size=256, num_attention_heads=4, num_query_groups=2, head_dim=64,
                 ffn_hidden_size=688, vocab_size=1024, dtype="fp32", mrope_section=(8, 12, 12), image_token_id=7,
                 vision=VisionConfig(num_layers=1, hidden_size=64, num_heads=2, ffn_hidden_size=96, patch_size=4,
                                     out_hidden_size=256)))
_reg(ModelConfig(name="tiny-glm4", num_layers=2, hidden_size=128, num_attention_heads=4, num_query_groups=2, head_dim=32,
                 ffn_hidden_size=256, vocab_size=512, qk_layernorm=False, qkv_bias=True, sandwich_norm=True, rotary_percent=0.5,
                 dtype="fp32"))
# GLM-4-9B-0414 / GLM-Z1 shape (trainer-side family like the other non-plain attention stacks)
_reg(ModelConfig(name="glm4-9b", num_layers=40, hidden_size=4096, num_attention_heads=32, num_query_groups=2, head_dim=128,
                 ffn_hidden_size=13696, vocab_size=151552, qk_layernorm=False, qkv_bias=True, sandwich_norm=True, rotary_percent=0.5,
                 rope_theta=1e4, rms_norm_eps=1e-5))
_reg(ModelConfig(name="tiny-qwen35", num_layers=4, hidden_size=128, num_attention_heads=4, num_query_groups=2, head_dim=32,
                 ffn_hidden_size=256, vocab_size=512, linear_attention_freq=4, attention_output_gate=True, rotary_percent=0.25,
                 dtype="fp32"))
_reg(ModelConfig(name="tiny-dsa", num_layers=2, hidden_size=128, num_attention_heads=4, num_query_groups=4, head_dim=32,
                 ffn_hidden_size=256, vocab_size=512, dsa_topk=8, dtype="fp32"))
_reg(ModelConfig(name="tiny-dsv3", num_layers=3, hidden_size=256, num_attention_heads=4, num_query_groups=2,
                 head_dim=64, ffn_hidden_size=688, vocab_size=1024, num_experts=8, moe_top_k=2, moe_ffn_hidden_size=128,
                 moe_first_dense_layers=1, moe_shared_expert_ffn=128, moe_router_score="sigmoid", moe_router_bias=True,
                 moe_routed_scaling_factor=2.5, dtype="fp32"))
# scripts/models/glm4.7-30B-A3B.sh: MLA + sigmoid-routed MoE with one shared expert and one leading dense layer
_reg(ModelConfig(name="glm4.7-30b-a3b", num_layers=47, hidden_size=2048, num_attention_heads=20, num_query_groups=20, head_dim=192,
                 ffn_hidden_size=10240, vocab_size=154880, qkv_bias=True, num_experts=64, moe_top_k=4, moe_ffn_hidden_size=1536,
                 moe_first_dense_layers=1, moe_shared_expert_ffn=1536, moe_router_score="sigmoid", moe_router_bias=True,
                 moe_router_bias_update_rate=0.0, moe_routed_scaling_factor=1.8, multi_latent_attention=True, dsa_q_lora=768,
                 dsa_kv_lora=512, dsa_nope=192, dsa_rope=64, dsa_v_head=256))
_reg(ModelConfig(name="tiny-mla", num_layers=2, hidden_size=128, num_attention_heads=4, num_query_groups=4, head_dim=32,
                 ffn_hidden_size=256, vocab_size=512, multi_latent_attention=True, dtype="fp32"))
_reg(ModelConfig(name="qwen3-1.7b", num_layers=28, hidden_size=2048, num_attention_heads=16, num_query_groups=8,
                 head_dim=128, ffn_hidden_size=6144, vocab_size=151936, tie_word_embeddings=True))
_reg(ModelConfig(name="qwen2.5-7b", num_layers=28, hidden_size=3584, num_attention_heads=28, num_query_groups=4,
                 head_dim=128, ffn_hidden_size=18944, vocab_size=152064, qk_layernorm=False, qkv_bias=True))
_reg(ModelConfig(name="qwen3-vl-8b", num_layers=36, hidden_size=4096, num_attention_heads=32, num_query_groups=8,
                 head_dim=128, ffn_hidden_size=12288, vocab_size=151936, rope_theta=5e6,
                 vision=VisionConfig(out_hidden_size=4096), mrope_section=(24, 20, 20), image_token_id=151655))
# Qwen3-VL family (scripts/models/qwen3-vl-*.sh of the reference): the language-model shapes of those recipes with the
# Qwen-VL tower of this package; the 30B-A3B variant is the MoE shape
_reg(ModelConfig(name="qwen3-vl-2b", num_layers=28, hidden_size=2048, num_attention_heads=16, num_query_groups=8,
                 head_dim=128, ffn_hidden_size=6144, vocab_size=151936, rope_theta=1e6,
                 vision=VisionConfig(out_hidden_size=2048), mrope_section=(24, 20, 20), image_token_id=151655))
_reg(ModelConfig(name="qwen3-vl-4b", num_layers=36, hidden_size=2560, num_attention_heads=32, num_query_groups=8,
                 head_dim=128, ffn_hidden_size=9728, vocab_size=151936, rope_theta=5e6, tie_word_embeddings=True,
                 vision=VisionConfig(out_hidden_size=2560), mrope_section=(24, 20, 20), image_token_id=151655))
_reg(ModelConfig(name="qwen3-vl-30b-a3b", num_layers=48, hidden_size=2048, num_attention_heads=32, num_query_groups=4,
                 head_dim=128, ffn_hidden_size=6144, vocab_size=151936, rope_theta=5e6, num_experts=128, moe_top_k=8,
                 moe_ffn_hidden_size=768, vision=VisionConfig(out_hidden_size=2048), mrope_section=(24, 20, 20),
                 image_token_id=151655))
_reg(ModelConfig(name="qwen3-omni-30b-a3b", num_layers=48, hidden_size=2048, num_attention_heads=32, num_query_groups=4,
                 head_dim=128, ffn_hidden_size=768, vocab_size=152064, rope_theta=1e6, num_experts=128, moe_top_k=8,
                 moe_ffn_hidden_size=768, vision=VisionConfig(out_hidden_size=2048), mrope_section=(24, 20, 20),
                 image_token_id=151655))
# Qwen3.5 family (scripts/models/qwen35-*.sh): hybrid stack - three Gated-DeltaNet layers, then one gated softmax-attention
# layer with 256-wide heads and rotary on their first quarter.  Trainer-side families (the rollout engine serves plain
# softmax attention).
_reg(ModelConfig(name="qwen3.5-9b", num_layers=32, hidden_size=4096, num_attention_heads=16, num_query_groups=4, head_dim=256,
                 ffn_hidden_size=12288, vocab_size=248320, rope_theta=1e7, attention_output_gate=True, rotary_percent=0.25,
                 layernorm_zero_centered=True, linear_attention_freq=4, gdn_k_heads=16, gdn_v_heads=32, gdn_head_dim=128))
_reg(ModelConfig(name="qwen3.5-35b-a3b", num_layers=40, hidden_size=2048, num_attention_heads=16, num_query_groups=2, head_dim=256,
                 ffn_hidden_size=512, vocab_size=248320, rope_theta=1e7, attention_output_gate=True, rotary_percent=0.25,
                 layernorm_zero_centered=True, linear_attention_freq=4, gdn_k_heads=16, gdn_v_heads=32, gdn_head_dim=128, num_experts=256, moe_top_k=8,
                 moe_ffn_hidden_size=512, moe_shared_expert_ffn=512, moe_shared_expert_gate=True))
# dots.ocr (scripts/models/dotsocr2.sh): a Qwen2.5-1.5B-shaped language model behind the dots tower (42 blocks of 1536, head_dim 128)
_reg(ModelConfig(name="dotsocr2", num_layers=28, hidden_size=1536, num_attention_heads=12, num_query_groups=2, head_dim=128,
                 ffn_hidden_size=8960, vocab_size=151936, qk_layernorm=False, qkv_bias=True, rope_theta=1e6,
                 vision=VisionConfig(num_layers=42, hidden_size=1536, num_heads=12, ffn_hidden_size=4224, temporal_patch_size=1,
                                     out_hidden_size=1536, patch_norm=True, post_trunk_norm=True, merger_layernorm=True,
                                     rms_norm_eps=1e-5),
                 mrope_section=(16, 24, 24), image_token_id=151655))
_reg(ModelConfig(name="qwen3-0.6b", num_layers=28, hidden_size=1024, num_attention_heads=16, num_query_groups=8,
                 head_dim=128, ffn_hidden_size=3072, vocab_size=151936, tie_word_embeddings=True))
_reg(ModelConfig(name="qwen3-4b", num_layers=36, hidden_size=2560, num_attention_heads=32, num_query_groups=8,
                 head_dim=128, ffn_hidden_size=9728, vocab_size=151936, tie_word_embeddings=True))
_reg(ModelConfig(name="qwen3-8b", num_layers=36, hidden_size=4096, num_attention_heads=32, num_query_groups=8,
                 head_dim=128, ffn_hidden_size=12288, vocab_size=151936))
_reg(ModelConfig(name="qwen3-32b", num_layers=64, hidden_size=5120, num_attention_heads=64, num_query_groups=8,
                 head_dim=128, ffn_hidden_size=25600, vocab_size=151936))
_reg(ModelConfig(name="qwen3-30b-a3b", num_layers=48, hidden_size=2048, num_attention_heads=32, num_query_groups=4,
                 head_dim=128, ffn_hidden_size=6144, vocab_size=151936, num_experts=128, moe_top_k=8,
                 moe_ffn_hidden_size=768))
_reg(ModelConfig(name="qwen2.5-vl-7b", num_layers=28, hidden_size=3584, num_attention_heads=28, num_query_groups=4,
                 head_dim=128, ffn_hidden_size=18944, vocab_size=152064, qk_layernorm=False, qkv_bias=True,
                 vision=VisionConfig(), mrope_section=(16, 24, 24), image_token_id=151655))
_reg(ModelConfig(name="llama3-8b", num_layers=32, hidden_size=4096, num_attention_heads=32, num_query_groups=8,
                 head_dim=128, ffn_hidden_size=14336, vocab_size=128256, qk_layernorm=False, rope_theta=5e5,
                 rms_norm_eps=1e-5))


def get_config(name: str, **overrides) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}")
    return replace(PRESETS[name], **overrides)
