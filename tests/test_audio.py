"""Audio tower + omni wrapper (CPU, tiny sizes)."""
import pytest
import torch

from relax_b200.data import multimodal as MM
from relax_b200.models.audio import AudioConfig, AudioEncoder, OmniModel
from relax_b200.models.config import get_config
from relax_b200.models.transformer import GPTModel


def _enc(out=256):
    return AudioEncoder(AudioConfig(n_mels=16, hidden_size=32, num_heads=2, intermediate_size=64, depth=2, out_hidden_size=out), seed=0)


def test_token_counts_match_the_preprocessor_and_clips_do_not_mix():
    enc = _enc()
    mels = [torch.randn(16, 100), torch.randn(16, 37), torch.randn(16, 8)]
    out, counts = enc(mels)
    assert counts == [MM.audio_token_count(100), MM.audio_token_count(37), MM.audio_token_count(8)]
    assert out.shape == (sum(counts), 256)
    alone, c2 = enc([mels[1]])
    assert c2 == [counts[1]] and torch.allclose(out[counts[0]:counts[0] + counts[1]], alone, atol=1e-5)


def test_omni_merges_audio_at_placeholders_and_backprops():
    cfg = get_config("tiny")
    enc = _enc(cfg.hidden_size)
    om = OmniModel(GPTModel(cfg, seed=0), audio=enc, audio_token_id=9)
    mel = torch.randn(16, 20)
    n = MM.audio_token_count(20)
    ids = MM.expand_placeholders([3, 9, 4, 5], 9, [n])
    toks = torch.tensor(ids)
    h = om(toks, torch.arange(len(ids)), torch.tensor([0, len(ids)], dtype=torch.int32), audio_mels=[mel])
    assert h.shape == (len(ids), cfg.hidden_size)
    h.square().mean().backward()
    assert enc.conv1_w.grad.abs().sum() > 0 and enc.merge_fc2.grad.abs().sum() > 0
    with pytest.raises(ValueError):
        om(torch.tensor([3, 9, 4]), torch.arange(3), torch.tensor([0, 3], dtype=torch.int32), audio_mels=[mel])
