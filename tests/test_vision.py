"""Vision encoder, M-RoPE position index, image-embedding merge, VL forward/backward (CPU, small sizes)."""
import pytest
import torch

from relax_b200.models.config import get_config
from relax_b200.models.transformer import GPTModel
from relax_b200.models.vision import (VisionConfig, VisionEncoder, VLModel, merge_image_embeddings, mrope_positions,
                                      vision_rope_tables)

VC = VisionConfig(patch_size=2, temporal_patch_size=1, in_channels=3, hidden_size=64, num_heads=4, intermediate_size=96,
                  depth=2, spatial_merge_size=2, out_hidden_size=256)


def test_mrope_positions_text_image_text():
    IMG = 99
    ids = [1, 2] + [IMG] * 6 + [3, 4]            # one image: t=1, 4x6 patches, merge 2 -> 2x3 tokens
    pos = mrope_positions(ids, [(1, 4, 6)], IMG, 2)
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3] and pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos[:, 8:].tolist() == [[5, 6]] * 3       # continues after max(t, h, w) = 3 past the image start
    with pytest.raises(ValueError):
        mrope_positions(ids, [(1, 4, 4)], IMG, 2)
    with pytest.raises(ValueError):
        mrope_positions([1, 2, 3], [(1, 4, 6)], IMG, 2)


def test_vision_rope_window_major_order():
    cos, sin = vision_rope_tables(torch.tensor([[1, 4, 4]]), 16, 10000.0, 2)
    assert cos.shape == (16, 8)
    # patch order: window (0,0) -> (r,c) = (0,0),(0,1),(1,0),(1,1); then window (0,1) -> columns 2,3
    ang_row = torch.atan2(sin[:, 0], cos[:, 0])      # frequency 0 of the row half has inv_freq 1
    ang_col = torch.atan2(sin[:, 4], cos[:, 4])
    assert torch.allclose(ang_row[:8], torch.tensor([0., 0., 1., 1., 0., 0., 1., 1.]), atol=1e-5)
    assert torch.allclose(ang_col[:8], torch.tensor([0., 1., 0., 1., 2., 3., 2., 3.]), atol=1e-5)


def test_encoder_shapes_and_image_independence():
    torch.manual_seed(0)
    enc = VisionEncoder(VC)
    g = torch.tensor([[1, 4, 4], [1, 2, 4]])
    n = 16 + 8
    px = torch.randn(n, VC.patch_dim)
    out = enc(px, g)
    assert out.shape == (n // 4, 256)
    # attention is per image: changing image 2 leaves image 1's tokens untouched
    px2 = px.clone()
    px2[16:] += 1.0
    out2 = enc(px2, g)
    assert torch.allclose(out[:4], out2[:4], atol=1e-6) and not torch.allclose(out[4:], out2[4:])


def test_vl_forward_backward_reaches_vision_weights():
    torch.manual_seed(0)
    cfg = get_config("tiny", mrope_section=[8, 12, 12])
    lm = GPTModel(cfg, seed=1)
    IMG = 7
    model = VLModel(lm, VisionEncoder(VisionConfig(**{**VC.__dict__, "out_hidden_size": cfg.hidden_size})), IMG)
    ids = [3, 4] + [IMG] * 4 + [5, 6, 8]
    tokens = torch.tensor(ids)
    pos = mrope_positions(ids, [(1, 4, 4)], IMG, 2)
    cu = torch.tensor([0, len(ids)], dtype=torch.int32)
    h = model(tokens, pos, cu, torch.randn(16, VC.patch_dim), torch.tensor([[1, 4, 4]]))
    lp, _ = lm.log_probs(h[:-1], tokens[1:], with_entropy=False)
    lp.sum().backward()
    assert model.vision.patch_embed.grad.abs().sum() > 0 and model.vision.blocks[0].qkv.grad.abs().sum() > 0
    with pytest.raises(ValueError):
        merge_image_embeddings(torch.zeros(9, 4), torch.zeros(3, 4), tokens, IMG)


def test_vision_branch_runs_as_dummy_when_only_peers_have_images():
    """The conditional-branch agreement makes a rank without images still produce (zero) vision gradients."""
    from relax_b200.models.vision import VLModel, VisionConfig, VisionEncoder
    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel

    class PeersHaveImages:            # stands in for the all-reduce MAX over the data-parallel group
        def run(self, active, branch, dummy):
            return branch() if active else dummy() * 0.0

    cfg = get_config("tiny", image_token_id=7)
    vc = VisionConfig(depth=1, hidden_size=32, num_heads=2, intermediate_size=64, patch_size=2, out_hidden_size=cfg.hidden_size)
    vl = VLModel(GPTModel(cfg, seed=0), VisionEncoder(vc), 7, branch_sync=PeersHaveImages())
    toks = torch.tensor([3, 4, 5, 6])
    h = vl(toks, torch.arange(4), torch.tensor([0, 4], dtype=torch.int32))
    h.sum().backward()
    g = vl.vision.patch_embed.grad
    assert g is not None and float(g.abs().sum()) == 0.0


def _tiny_vl():
    from relax_b200.models.config import VisionConfig, get_config

    return get_config("tiny", vision=VisionConfig(num_layers=1, hidden_size=64, num_heads=2, ffn_hidden_size=96, patch_size=4,
                                                  out_hidden_size=256), mrope_section=(8, 12, 12), image_token_id=7)


def test_engine_takes_images_and_matches_the_trainer():
    """Image prompts through the rollout engine (patches -> tower -> placeholder rows, M-RoPE ids, shifted decode
    positions, host-driven and windowed decode) give the log-probs the trainer computes for the same samples."""
    import torch

    from relax_b200.rollout.data_source import RolloutDataSource, SyntheticImagePromptDataset
    from relax_b200.rollout.engine import RolloutEngine, SamplingParams
    from relax_b200.train.actor import TrainActor, TrainConfig
    from relax_b200.weight_sync.plan import TrainerLayout
    from relax_b200.weight_sync.sync import WeightSync

    cfg = _tiny_vl()
    actor = TrainActor(cfg, TrainConfig(), seed=0, with_optimizer=False)
    assert any(n.startswith("vision.") for n, _ in actor.model.named_parameters())
    ds = SyntheticImagePromptDataset(3, 5, cfg.vocab_size, cfg.image_token_id, grid_hw=(4, 6), patch_dim=3 * 2 * 4 * 4, seed=1)
    groups = RolloutDataSource(ds, 2).get_samples(3)
    flat = [s for g in groups for s in g]
    flat[2].multimodal_train_inputs = flat[3].multimodal_train_inputs = None     # one text-only group in the batch
    for s in flat[2:4]:
        s.tokens = [t for t in s.tokens if t != cfg.image_token_id]
    outs = {}
    for windowed in (False, True):
        eng = RolloutEngine(cfg, device="cpu", dtype=torch.float32, num_kv_blocks=128, block_size=8, windowed_decode=windowed,
                            decode_window=4)
        WeightSync(cfg, TrainerLayout(), 1, [0], [0]).update_weights(dict(actor.named_local_params()), eng.weights, eng, 1)
        eng.attach_vision(actor.model.vision)
        res = eng.generate([s.tokens for s in flat], SamplingParams(max_new_tokens=7, temperature=1.0),
                           group_keys=[s.group_index for s in flat], images=[s.multimodal_train_inputs for s in flat])
        outs[windowed] = res
        assert res[0].pos_delta < 0 and res[2].pos_delta == 0      # 6 placeholders advance the position by max(2, 3) = 3
        batch = {"tokens": [r.prompt + r.output for r in res], "response_lengths": [len(r.output) for r in res],
                 "multimodal_train_inputs": [s.multimodal_train_inputs for s in flat]}
        lp = actor.compute_log_prob(batch)["log_probs"]
        for r, l in zip(res, lp):
            assert torch.allclose(torch.tensor(r.logprobs), l, atol=2e-4), (windowed, r.rid)
    assert [r.output for r in outs[False]] == [r.output for r in outs[True]]


def test_vl_training_step_moves_the_tower():
    import torch

    from relax_b200.train.actor import TrainActor, TrainConfig

    cfg = _tiny_vl()
    actor = TrainActor(cfg, TrainConfig(), seed=0)
    g = torch.Generator().manual_seed(0)
    n_img = 2 * 2 // 4 * 1 or 1
    toks, mm = [], []
    for i in range(4):
        p = torch.randint(8, cfg.vocab_size, (6,), generator=g).tolist()
        toks.append(p[:3] + [cfg.image_token_id] * 1 + p[3:] + torch.randint(8, cfg.vocab_size, (5,), generator=g).tolist())
        mm.append({"pixel_patches": torch.randn(4, 3 * 2 * 4 * 4, generator=g), "grid_thw": torch.tensor([[1, 2, 2]])})
    batch = {"tokens": toks, "response_lengths": [5] * 4, "rewards": [1.0, 0.0, 0.5, 0.2], "multimodal_train_inputs": mm,
             "rollout_log_probs": [[-1.0] * 5] * 4, "loss_masks": [[1] * 5] * 4, "group_index": [0, 0, 1, 1]}
    before = actor.model.vision.patch_embed.detach().clone()
    m = actor.train(0, batch)
    assert m["grad_norm"] > 0
    assert not torch.equal(before, actor.model.vision.patch_embed.detach())


def test_colocated_grpo_with_images_end_to_end():
    """Config-3 shape on the CPU: synthetic image prompts -> engine (tower at prefill) -> rewards -> reference and
    old-policy forward -> GRPO update of language model and tower -> weight sync, two steps."""
    import math

    import torch

    from relax_b200.algo.loss import LossConfig
    from relax_b200.orchestration.colocate import ColocateConfig, ColocatedGRPO
    from relax_b200.train.actor import TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    torch.manual_seed(0)
    cfg = ColocateConfig(
        model=_tiny_vl(),
        train=TrainConfig(advantage_estimator="grpo", n_samples_per_prompt=4, global_batch_size=16, max_tokens_per_gpu=2048,
                          loss=LossConfig(eps_clip=0.2, use_kl_loss=True, kl_loss_coef=0.001, kl_loss_type="k1"),
                          optim=OptimizerConfig(lr=1e-4, clip_grad=1.0)),
        rollout_batch_size=4, prompt_len=32, max_response_len=12, temperature=1.0, rm_type="parity", eos_token_id=3,
        seed=0, rollout_seed=42)
    run = ColocatedGRPO(cfg)
    tower0 = run.actor.model.vision.patch_embed.detach().clone()
    for _ in range(2):
        m = run.step()
        assert math.isfinite(m["loss"]) and m["grad_norm"] > 0
        assert m["train_rollout_logprob_abs_diff"] < 1e-3
    assert not torch.equal(tower0, run.actor.model.vision.patch_embed.detach())
    run.close()


def test_vision_language_checkpoint_names_round_trip(tmp_path):
    """A vision-language model saved under Qwen2.5-VL's Hugging Face names (decoder under ``model.language_model.*``, tower
    under ``model.visual.*`` with the convolution-shaped patch embedding and un-padded MLP width) loads back exactly."""
    import torch

    from relax_b200.checkpoint import hf as HF
    from relax_b200.models.vision import load_vision_from_hf, vision_state_to_hf
    from relax_b200.train.actor import TrainActor, TrainConfig

    cfg = _tiny_vl()
    a = TrainActor(cfg, TrainConfig(), seed=1, with_optimizer=False)
    g = torch.Generator().manual_seed(0)
    for n, p in a.model.named_parameters():      # biases start at zero: give everything a value
        p.data.copy_(torch.randn(p.shape, generator=g) * 0.05)
    for b in a.model.vision.blocks:              # the width padding is structurally zero
        b.fc1.data[b.f:b.f_pad] = 0; b.fc1.data[b.f_pad + b.f:] = 0; b.fc2.data[:, b.f:] = 0
        b.fc1_bias.data[b.f:b.f_pad] = 0; b.fc1_bias.data[b.f_pad + b.f:] = 0
    tower = vision_state_to_hf(a.model.vision, "model.visual.")
    v = cfg.vision
    assert tower["model.visual.patch_embed.proj.weight"].shape == (v.hidden_size, v.in_channels, v.temporal_patch_size, v.patch_size, v.patch_size)
    assert tower["model.visual.blocks.0.mlp.gate_proj.weight"].shape[0] == v.ffn_hidden_size
    lm = HF.convert_state_to_hf(cfg, {n: p.detach() for n, p in a.model.named_parameters() if not n.startswith("vision.")})
    state = {("model.language_model." + k[len("model."):] if k.startswith("model.") else k): t for k, t in lm.items()}
    state.update(tower)
    d = str(tmp_path / "vl")
    HF.save_hf_checkpoint(d, cfg, state)
    b = TrainActor(cfg, TrainConfig(), seed=2, with_optimizer=False)
    assert HF.load_hf_into_model(d, cfg, b.ps, b.model) == []
    for (n, p), (_, q) in zip(a.model.named_parameters(), b.model.named_parameters()):
        assert torch.equal(p, q), n
    # a text-only checkpoint leaves the tower alone unless strict
    import pytest

    with pytest.raises(KeyError):
        load_vision_from_hf(b.model.vision, lm, strict=True)


def test_dots_ocr_tower_variant_matches_a_plain_statement():
    """The dots.ocr tower: RMSNorm on the patch embeddings and after the trunk, LayerNorm in front of the merger, one
    temporal slice per patch - against a direct PyTorch statement of the same network."""
    import math

    import torch
    import torch.nn.functional as F

    from relax_b200 import ops
    from relax_b200.models.config import get_config
    from relax_b200.models.vision import VisionConfig, VisionEncoder, vision_config_from_model, vision_rope_tables

    full = vision_config_from_model(get_config("dotsocr2"))
    assert full.depth == 42 and full.head_dim == 128 and full.patch_norm and full.post_trunk_norm and full.merger_layernorm
    cfg = VisionConfig(patch_size=4, temporal_patch_size=1, hidden_size=64, num_heads=2, intermediate_size=96, depth=2,
                       out_hidden_size=48, rms_norm_eps=1e-5, patch_norm=True, post_trunk_norm=True, merger_layernorm=True)
    enc = VisionEncoder(cfg, seed=4)
    g = torch.Generator().manual_seed(1)
    for p in enc.parameters():
        p.data.add_(torch.randn(p.shape, generator=g) * 0.05)
    grid = torch.tensor([[1, 4, 6]])
    px = torch.randn(24, cfg.patch_dim, generator=g)
    got = enc(px, grid)

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    x = rms(px @ enc.patch_embed.t(), enc.patch_norm)
    cos, sin = vision_rope_tables(grid, cfg.head_dim, cfg.rope_theta, cfg.spatial_merge_size)
    for b in enc.blocks:
        y = rms(x, b.norm1)
        qkv = (y @ b.qkv.t() + b.qkv_bias).view(-1, 3, cfg.num_heads, cfg.head_dim)
        q, k, v = ops.apply_rope(qkv[:, 0], cos, sin), ops.apply_rope(qkv[:, 1], cos, sin), qkv[:, 2]
        att = torch.softmax(torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(cfg.head_dim), -1)
        o = torch.einsum("hqk,khd->qhd", att, v).reshape(x.shape[0], -1)
        x = x + o @ b.proj.t() + b.proj_bias
        y = rms(x, b.norm2)
        gu = y @ b.fc1.t() + b.fc1_bias
        x = x + (F.silu(gu[:, :b.f_pad]) * gu[:, b.f_pad:]) @ b.fc2.t() + b.fc2_bias
    x = rms(x, enc.post_trunk_norm)
    x = F.layer_norm(x, (cfg.hidden_size,), enc.merger_norm, enc.merger_norm_bias, 1e-6).view(-1, cfg.hidden_size * 4)
    want = F.gelu(x @ enc.merger_fc1.t() + enc.merger_fc1_bias) @ enc.merger_fc2.t() + enc.merger_fc2_bias
    assert torch.allclose(got, want, atol=2e-5), (got - want).abs().max()
