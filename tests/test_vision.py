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
