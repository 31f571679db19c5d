"""Image / video / audio preprocessing for the vision-language and omni model families.

Covers the reference's multimodal helpers (relax/utils/multimodal/: ``image_utils.py`` smart resize + loaders,
``video_utils.py`` frame-count and per-frame pixel budget, ``audio_utils.py`` loaders, ``process.py`` message
scanning, ``stats.py`` token counts, ``config.py`` limits).  Everything is plain torch / numpy on the host; the
output layout is the one :class:`relax_b200.models.vision.VisionEncoder` consumes: patches in
merge-window-major order, ``[N, C * temporal_patch * patch * patch]``, with a ``grid_thw`` row per item.

Decoding of containers is delegated to what the image has (PIL for images, ``.npy`` / raw tensors for
video frames and audio, WAV through the standard library); there is no codec dependency.
"""
from __future__ import annotations

import base64
import io
import math
import wave
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


@dataclass
class MultimodalConfig:
    """Limits in *merged* tokens (one token = ``merge x merge`` patches), as the reference's config.py."""
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    image_min_tokens: int = 4
    image_max_tokens: int = 16384
    video_min_tokens: int = 128
    video_max_tokens: int = 768          # per frame
    video_total_tokens: int = 24576      # whole clip
    video_fps: float = 2.0
    video_min_frames: int = 4
    video_max_frames: int = 768
    frame_factor: int = 2
    audio_sample_rate: int = 16000
    audio_n_mels: int = 128
    audio_n_fft: int = 400
    audio_hop: int = 160
    max_aspect_ratio: float = 200.0

    @property
    def factor(self) -> int:
        return self.patch_size * self.spatial_merge_size


# --------------------------------------------------------------------------- sizes
def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int, max_ratio: float = 200.0):
    """Target size with both sides multiples of ``factor``, the pixel count inside ``[min_pixels, max_pixels]``
    and the aspect ratio kept as closely as rounding allows (relax/utils/multimodal/image_utils.py :31-83)."""
    if min(height, width) <= 0:
        raise ValueError("empty image")
    if max(height, width) / min(height, width) > max_ratio:
        raise ValueError(f"aspect ratio above {max_ratio}")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def image_target_size(height: int, width: int, cfg: MultimodalConfig):
    f2 = cfg.factor * cfg.factor
    return smart_resize(height, width, cfg.factor, cfg.image_min_tokens * f2, cfg.image_max_tokens * f2, cfg.max_aspect_ratio)


def smart_video_nframes(total_frames: int, source_fps: float, cfg: MultimodalConfig, fps: Optional[float] = None,
                        nframes: Optional[int] = None) -> int:
    """Frames to sample: ``duration * fps`` clamped to the configured range and the clip length, rounded to a
    multiple of ``frame_factor`` (relax/utils/multimodal/video_utils.py :98-127)."""
    ff = cfg.frame_factor
    if nframes is not None:
        n = round(nframes / ff) * ff
    else:
        want = total_frames / max(source_fps, 1e-6) * (fps or cfg.video_fps)
        lo = math.ceil(cfg.video_min_frames / ff) * ff
        hi = math.floor(min(cfg.video_max_frames, total_frames) / ff) * ff
        n = math.floor(min(max(want, lo), max(hi, ff)) / ff) * ff
    n = max(ff, n)
    if n > total_frames and total_frames >= ff:
        n = total_frames // ff * ff
    return int(n)


def video_target_size(nframes: int, height: int, width: int, cfg: MultimodalConfig):
    """Per-frame size under the clip-wide token budget (:56-96 of the reference's video_utils.py)."""
    f2 = cfg.factor * cfg.factor
    per_frame = cfg.video_total_tokens * cfg.temporal_patch_size // max(1, nframes)
    max_tok = max(cfg.video_min_tokens, min(cfg.video_max_tokens, per_frame))
    return smart_resize(height, width, cfg.factor, cfg.video_min_tokens * f2, max_tok * f2, cfg.max_aspect_ratio)


def sample_frame_indices(total_frames: int, n: int) -> List[int]:
    return [int(round(i)) for i in np.linspace(0, total_frames - 1, n)]


# --------------------------------------------------------------------------- pixels -> patches
def _resize(img: torch.Tensor, h: int, w: int) -> torch.Tensor:
    """``img [.., C, H, W]`` float in [0, 1] -> bicubic, antialiased."""
    lead = img.shape[:-3]
    x = img.reshape(-1, *img.shape[-3:]).float()
    x = F.interpolate(x, size=(h, w), mode="bicubic", align_corners=False, antialias=True).clamp_(0, 1)
    return x.reshape(*lead, *x.shape[-3:])


def _normalise(x: torch.Tensor) -> torch.Tensor:
    mean = torch.tensor(CLIP_MEAN, dtype=x.dtype).view(-1, 1, 1)
    std = torch.tensor(CLIP_STD, dtype=x.dtype).view(-1, 1, 1)
    return (x - mean) / std


def frames_to_patches(frames: torch.Tensor, cfg: MultimodalConfig):
    """``frames [T, C, H, W]`` (T a multiple of the temporal patch; H, W multiples of ``factor``) ->
    ``(patches [N, C * tp * P * P], (t, h, w))`` with the ``merge x merge`` neighbours adjacent."""
    T, C, H, W = frames.shape
    P, m, tp = cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size
    assert T % tp == 0 and H % (P * m) == 0 and W % (P * m) == 0
    gt, gh, gw = T // tp, H // P, W // P
    x = frames.reshape(gt, tp, C, gh // m, m, P, gw // m, m, P)
    #            0   1   2   3       4  5   6       7  8
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)   # gt, gh/m, gw/m, m, m, C, tp, P, P
    return x.reshape(gt * gh * gw, C * tp * P * P).contiguous(), (gt, gh, gw)


def process_image(img, cfg: Optional[MultimodalConfig] = None):
    """One image (PIL image, ``[H, W, C]`` uint8 array or ``[C, H, W]`` float tensor) -> ``(patches, grid_thw)``.
    The single frame is repeated over the temporal patch, as the Qwen2-VL processor does."""
    cfg = cfg or MultimodalConfig()
    x = to_chw_float(img)
    h, w = image_target_size(x.shape[1], x.shape[2], cfg)
    x = _normalise(_resize(x, h, w))
    return frames_to_patches(x[None].repeat(cfg.temporal_patch_size, 1, 1, 1), cfg)


def process_video(frames, source_fps: float = 30.0, cfg: Optional[MultimodalConfig] = None, fps: Optional[float] = None,
                  nframes: Optional[int] = None):
    """``frames [T, C, H, W]`` (or ``[T, H, W, C]`` uint8) -> ``(patches, grid_thw, sampled_indices)``."""
    cfg = cfg or MultimodalConfig()
    v = torch.as_tensor(np.asarray(frames)) if not torch.is_tensor(frames) else frames
    if v.shape[-1] in (1, 3) and v.shape[1] not in (1, 3):
        v = v.permute(0, 3, 1, 2)
    v = v.float() / 255.0 if v.dtype == torch.uint8 else v.float()
    n = smart_video_nframes(v.shape[0], source_fps, cfg, fps, nframes)
    idx = sample_frame_indices(v.shape[0], n)
    v = v[idx]
    pad = (-v.shape[0]) % cfg.temporal_patch_size
    if pad:
        v = torch.cat([v, v[-1:].repeat(pad, 1, 1, 1)])
    h, w = video_target_size(v.shape[0], v.shape[2], v.shape[3], cfg)
    p, g = frames_to_patches(_normalise(_resize(v, h, w)), cfg)
    return p, g, idx


def to_chw_float(img) -> torch.Tensor:
    if torch.is_tensor(img):
        x = img
    else:
        arr = np.asarray(img.convert("RGB") if hasattr(img, "convert") else img)
        x = torch.from_numpy(np.ascontiguousarray(arr))
    if x.dim() == 2:
        x = x[None].repeat(3, 1, 1) if x.dtype != torch.uint8 else x[..., None].repeat(1, 1, 3)
    if x.shape[-1] in (1, 3, 4) and x.shape[0] not in (1, 3):
        x = x[..., :3].permute(2, 0, 1)
    x = x.float() / 255.0 if x.dtype == torch.uint8 else x.float()
    if x.shape[0] == 1:
        x = x.repeat(3, 1, 1)
    return x


# --------------------------------------------------------------------------- loaders
def decode_data_uri(uri: str) -> bytes:
    """``data:<mime>;base64,<payload>`` -> bytes (relax/utils/multimodal/image_utils.py :203-215)."""
    if not uri.startswith("data:") or "," not in uri:
        raise ValueError("not a data URI")
    head, payload = uri.split(",", 1)
    return base64.b64decode(payload) if head.endswith(";base64") else payload.encode()


def load_image(src):
    """Path, ``file://`` URL, data URI, bytes, PIL image, array or tensor -> ``[C, H, W]`` float tensor.
    Remote URLs are refused: the data plane never opens network connections during preprocessing."""
    from PIL import Image

    if isinstance(src, (bytes, bytearray)):
        return to_chw_float(Image.open(io.BytesIO(src)))
    if isinstance(src, str):
        if src.startswith("data:"):
            return to_chw_float(Image.open(io.BytesIO(decode_data_uri(src))))
        if src.startswith(("http://", "https://")):
            raise ValueError("remote image URLs are not fetched; download the dataset first")
        path = src[7:] if src.startswith("file://") else src
        if path.endswith(".npy"):
            return to_chw_float(np.load(path))
        return to_chw_float(Image.open(path))
    return to_chw_float(src)


def load_audio(src, cfg: Optional[MultimodalConfig] = None) -> torch.Tensor:
    """WAV path / bytes, ``.npy`` path, ``(array, rate)`` pair or 1-D array at the target rate -> mono float
    waveform at ``cfg.audio_sample_rate`` (relax/utils/multimodal/audio_utils.py :73-113)."""
    cfg = cfg or MultimodalConfig()
    rate = cfg.audio_sample_rate
    if isinstance(src, tuple):
        wav, rate = torch.as_tensor(np.asarray(src[0]), dtype=torch.float32), int(src[1])
    elif isinstance(src, (bytes, bytearray)) or (isinstance(src, str) and not src.endswith(".npy")):
        with wave.open(io.BytesIO(src) if not isinstance(src, str) else src, "rb") as f:
            rate, nch, width = f.getframerate(), f.getnchannels(), f.getsampwidth()
            raw = f.readframes(f.getnframes())
        dt = {1: np.uint8, 2: np.int16, 4: np.int32}[width]
        a = np.frombuffer(raw, dtype=dt).astype(np.float32)
        a = (a - 128.0) / 128.0 if width == 1 else a / float(2 ** (8 * width - 1))
        wav = torch.from_numpy(a.reshape(-1, nch).mean(1))
    elif isinstance(src, str):
        wav = torch.as_tensor(np.load(src), dtype=torch.float32)
    else:
        wav = torch.as_tensor(np.asarray(src), dtype=torch.float32)
    if wav.dim() > 1:
        wav = wav.mean(0 if wav.shape[0] < wav.shape[-1] else -1)
    if rate != cfg.audio_sample_rate:
        n = int(round(wav.numel() * cfg.audio_sample_rate / rate))
        wav = F.interpolate(wav[None, None], size=n, mode="linear", align_corners=False)[0, 0]
    return wav


# --------------------------------------------------------------------------- audio features
def _hz_to_mel(f):
    f = np.asarray(f, dtype=np.float64)
    lin = f / (200.0 / 3)
    log = 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0)
    return np.where(f >= 1000.0, log, lin)


def _mel_to_hz(m):
    m = np.asarray(m, dtype=np.float64)
    lin = m * (200.0 / 3)
    log = 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0))
    return np.where(m >= 15.0, log, lin)


def mel_filterbank(n_mels: int, n_fft: int, rate: int) -> torch.Tensor:
    """Slaney-normalised triangular filters ``[n_mels, n_fft // 2 + 1]`` (the Whisper front end)."""
    freqs = np.linspace(0, rate / 2, n_fft // 2 + 1)
    pts = _mel_to_hz(np.linspace(_hz_to_mel(0.0), _hz_to_mel(rate / 2), n_mels + 2))
    fb = np.zeros((n_mels, freqs.size))
    for i in range(n_mels):
        lo, c, hi = pts[i], pts[i + 1], pts[i + 2]
        up, down = (freqs - lo) / max(c - lo, 1e-10), (hi - freqs) / max(hi - c, 1e-10)
        fb[i] = np.maximum(0, np.minimum(up, down)) * (2.0 / (hi - lo))
    return torch.from_numpy(fb).float()


def log_mel_spectrogram(wav: torch.Tensor, cfg: Optional[MultimodalConfig] = None) -> torch.Tensor:
    """``[n_mels, frames]`` log-mel features: Hann STFT power -> mel -> log10, floored 8 dB under the peak and
    mapped to roughly [-1, 1]; one frame per ``audio_hop`` samples."""
    cfg = cfg or MultimodalConfig()
    win = torch.hann_window(cfg.audio_n_fft)
    spec = torch.stft(wav.float(), cfg.audio_n_fft, cfg.audio_hop, window=win, return_complex=True)
    power = spec[..., :-1].abs() ** 2
    mel = mel_filterbank(cfg.audio_n_mels, cfg.audio_n_fft, cfg.audio_sample_rate) @ power
    lg = torch.clamp(mel, min=1e-10).log10()
    lg = torch.maximum(lg, lg.max() - 8.0)
    return (lg + 4.0) / 4.0


def audio_token_count(n_frames: int) -> int:
    """Tokens the audio tower emits for ``n_frames`` mel frames (a stride-2 convolution, then pairs of frames merged)."""
    after = (n_frames - 1) // 2 + 1
    return (after - 2) // 2 + 1 if after >= 2 else 1


def smart_audio_nframes(duration_s: float, cfg: Optional[MultimodalConfig] = None) -> int:
    cfg = cfg or MultimodalConfig()
    return int(duration_s * cfg.audio_sample_rate) // cfg.audio_hop


# --------------------------------------------------------------------------- messages
def is_multimodal_element(e: Dict[str, Any]) -> bool:
    return isinstance(e, dict) and (e.get("type") in ("image", "image_url", "video", "audio")
                                    or any(k in e for k in ("image", "image_url", "video", "audio")))


def extract_vision_info(messages: Sequence[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """All image / video / audio parts of a chat, in order (relax/utils/multimodal/process.py :28-50)."""
    out = []
    for msg in messages:
        content = msg.get("content")
        if isinstance(content, list):
            out.extend(e for e in content if is_multimodal_element(e))
    return out


def process_multimodal_info(messages: Sequence[Dict[str, Any]], cfg: Optional[MultimodalConfig] = None) -> Dict[str, Any]:
    """Preprocess every media part of a chat.  Returns ``pixel_values`` / ``image_grid_thw``,
    ``pixel_values_videos`` / ``video_grid_thw`` and ``audio_features`` / ``audio_lengths`` (keys absent when the
    chat has no such part), plus ``num_tokens`` per kind for the placeholder expansion."""
    cfg = cfg or MultimodalConfig()
    img_p, img_g, vid_p, vid_g, aud, aud_len = [], [], [], [], [], []
    for e in extract_vision_info(messages):
        if "image" in e or "image_url" in e:
            src = e.get("image", e.get("image_url"))
            if isinstance(src, dict):
                src = src.get("url")
            p, g = process_image(load_image(src), cfg)
            img_p.append(p)
            img_g.append(g)
        elif "video" in e:
            v = e["video"]
            if isinstance(v, (list, tuple)) and not torch.is_tensor(v):
                v = torch.stack([load_image(f) for f in v])
            elif isinstance(v, str):
                v = np.load(v)
            p, g, _ = process_video(v, e.get("source_fps", 30.0), cfg, e.get("fps"), e.get("nframes"))
            vid_p.append(p)
            vid_g.append(g)
        elif "audio" in e:
            f = log_mel_spectrogram(load_audio(e["audio"], cfg), cfg)
            aud.append(f)
            aud_len.append(f.shape[1])
    out: Dict[str, Any] = {"num_tokens": {}}
    m2 = cfg.spatial_merge_size ** 2
    if img_p:
        out["pixel_values"] = torch.cat(img_p)
        out["image_grid_thw"] = torch.tensor(img_g, dtype=torch.int64)
        out["num_tokens"]["image"] = [t * h * w // m2 for t, h, w in img_g]
    if vid_p:
        out["pixel_values_videos"] = torch.cat(vid_p)
        out["video_grid_thw"] = torch.tensor(vid_g, dtype=torch.int64)
        out["num_tokens"]["video"] = [t * h * w // m2 for t, h, w in vid_g]
    if aud:
        out["audio_features"] = aud
        out["audio_lengths"] = aud_len
        out["num_tokens"]["audio"] = [audio_token_count(n) for n in aud_len]
    return out


def get_multimodal_token_counts(mm: Optional[Dict[str, Any]]) -> Dict[str, int]:
    """Totals for logging (relax/utils/multimodal/stats.py :52-60)."""
    nt = (mm or {}).get("num_tokens", {})
    return {f"{k}_tokens": int(sum(nt.get(k, []))) for k in ("image", "video", "audio")} | {
        "num_images": len(nt.get("image", [])), "num_videos": len(nt.get("video", [])), "num_audios": len(nt.get("audio", []))}


def expand_placeholders(input_ids: Sequence[int], token_id: int, counts: Sequence[int]) -> List[int]:
    """Replace the i-th occurrence of ``token_id`` by ``counts[i]`` copies (what the HF processors do to the
    ``<|image_pad|>`` placeholder before the ids reach the model)."""
    out, i = [], 0
    for t in input_ids:
        if t == token_id:
            if i >= len(counts):
                raise ValueError("more placeholders than media items")
            out.extend([token_id] * counts[i])
            i += 1
        else:
            out.append(t)
    if i != len(counts):
        raise ValueError("fewer placeholders than media items")
    return out
