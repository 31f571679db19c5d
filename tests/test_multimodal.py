"""Image / video / audio preprocessing (CPU)."""
import base64
import io
import math
import wave

import numpy as np
import pytest
import torch

from relax_b200.data import multimodal as MM
from relax_b200.models.vision import VisionConfig, VisionEncoder


def test_smart_resize_bounds_and_factor():
    h, w = MM.smart_resize(1000, 700, 28, 4 * 784, 256 * 784)
    assert h % 28 == 0 and w % 28 == 0 and 4 * 784 <= h * w <= 256 * 784
    assert abs(h / w - 1000 / 700) < 0.1
    h, w = MM.smart_resize(20, 30, 28, 4 * 784, 256 * 784)           # upscaled to the minimum
    assert h * w >= 4 * 784 and h % 28 == 0
    assert MM.smart_resize(280, 280, 28, 784, 10 ** 9) == (280, 280)  # already fine
    with pytest.raises(ValueError):
        MM.smart_resize(10, 5000, 28, 784, 10 ** 9)


def test_patch_layout_matches_vision_encoder_contract():
    cfg = MM.MultimodalConfig(patch_size=2, spatial_merge_size=2, temporal_patch_size=2, image_min_tokens=1, image_max_tokens=64)
    fr = torch.arange(2 * 3 * 8 * 8, dtype=torch.float32).reshape(2, 3, 8, 8)
    p, (t, h, w) = MM.frames_to_patches(fr, cfg)
    assert (t, h, w) == (1, 4, 4) and p.shape == (16, 3 * 2 * 2 * 2)
    # patch 1 is the right neighbour of patch 0 inside the first 2x2 merge window; patch 2 is below patch 0
    def patch(r, c):
        return fr[:, :, 2 * r:2 * r + 2, 2 * c:2 * c + 2].permute(1, 0, 2, 3).reshape(-1)
    assert torch.equal(p[0], patch(0, 0)) and torch.equal(p[1], patch(0, 1)) and torch.equal(p[2], patch(1, 0))
    assert torch.equal(p[4], patch(0, 2))    # next window to the right
    # and the encoder accepts it
    vc = VisionConfig(depth=1, hidden_size=32, num_heads=2, intermediate_size=64, patch_size=2, spatial_merge_size=2,
                      temporal_patch_size=2, out_hidden_size=16)
    enc = VisionEncoder(vc)
    out = enc(p, torch.tensor([[t, h, w]]))
    assert out.shape == (4, 16)


def test_process_image_and_data_uri_roundtrip():
    from PIL import Image

    rng = np.random.default_rng(0)
    arr = rng.integers(0, 255, (60, 90, 3), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="PNG")
    uri = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    img = MM.load_image(uri)
    assert img.shape == (3, 60, 90) and torch.allclose(img, torch.from_numpy(arr).permute(2, 0, 1).float() / 255)
    cfg = MM.MultimodalConfig()
    p, (t, h, w) = MM.process_image(img, cfg)
    assert t == 1 and p.shape == (h * w, 3 * 2 * 14 * 14) and h % 2 == 0 and w % 2 == 0
    with pytest.raises(ValueError):
        MM.load_image("https://example.com/x.png")


def test_video_frame_count_and_budget():
    cfg = MM.MultimodalConfig(video_fps=2.0, video_min_frames=4, video_max_frames=16)
    assert MM.smart_video_nframes(300, 30.0, cfg) == 16            # 10 s * 2 fps = 20 -> capped
    assert MM.smart_video_nframes(90, 30.0, cfg) == 6
    assert MM.smart_video_nframes(30, 30.0, cfg) == 4              # floor at the minimum
    assert MM.smart_video_nframes(300, 30.0, cfg, nframes=7) in (6, 8)
    cfg2 = MM.MultimodalConfig(video_total_tokens=64, video_min_tokens=4, video_max_tokens=64, video_min_frames=2)
    frames = torch.rand(8, 3, 56, 84)
    p, (t, h, w), idx = MM.process_video(frames, 4.0, cfg2)
    assert t == len(idx) // 2 and p.shape[0] == t * h * w and idx[0] == 0 and idx[-1] == 7
    assert h * w // 4 <= 64


def test_log_mel_of_a_tone_peaks_at_the_right_band():
    cfg = MM.MultimodalConfig()
    t = torch.arange(16000) / 16000.0
    wav = torch.sin(2 * math.pi * 1000.0 * t)
    buf = io.BytesIO()
    with wave.open(buf, "wb") as f:
        f.setnchannels(1); f.setsampwidth(2); f.setframerate(8000)
        f.writeframes((wav[::2] * 32000).to(torch.int16).numpy().tobytes())
    w8 = MM.load_audio(buf.getvalue(), cfg)              # resampled 8 kHz -> 16 kHz
    assert abs(w8.numel() - 16000) <= 2
    mel = MM.log_mel_spectrogram(wav, cfg)
    assert mel.shape == (128, 100)
    fb = MM.mel_filterbank(128, 400, 16000)
    centre = fb[:, round(1000 / (16000 / 400))].argmax()
    assert abs(int(mel.mean(1).argmax()) - int(centre)) <= 1
    assert MM.audio_token_count(100) == 25 and MM.smart_audio_nframes(1.0, cfg) == 100


def test_process_messages_and_placeholders():
    img = (np.random.default_rng(1).random((56, 56, 3)) * 255).astype(np.uint8)
    msgs = [{"role": "user", "content": [{"type": "text", "text": "what"}, {"type": "image", "image": img},
                                          {"type": "audio", "audio": (np.zeros(3200, dtype=np.float32), 16000)}]},
            {"role": "assistant", "content": "a cat"}]
    assert len(MM.extract_vision_info(msgs)) == 2
    out = MM.process_multimodal_info(msgs)
    n_img = out["num_tokens"]["image"][0]
    assert out["pixel_values"].shape[0] == n_img * 4 and out["image_grid_thw"].tolist() == [[1, 4, 4]]
    assert out["audio_lengths"] == [20]
    ids = MM.expand_placeholders([1, 99, 2], 99, [n_img])
    assert ids.count(99) == n_img
    st = MM.get_multimodal_token_counts(out)
    assert st["image_tokens"] == n_img and st["num_audios"] == 1 and st["num_videos"] == 0
    with pytest.raises(ValueError):
        MM.expand_placeholders([1, 2], 99, [3])
