"""Checkpoint conversion command line (the reference's ``scripts/tools``: ``convert_torch_dist_to_hf_bridge.py``,
``convert_hf_to_fp8.py``, ``convert_fp8_to_bf16.py``, ``convert_hf_to_int4.py``, ``convert_moe_int4_to_bf16.py``,
``merge_lora_adapter_to_hf.py``):

    python -m relax_b200.checkpoint.convert dist2hf  --model-name qwen3-8b --load ckpt/ --out hf/
    python -m relax_b200.checkpoint.convert hf2dist  --model-name qwen3-8b --load hf/ --out ckpt/
    python -m relax_b200.checkpoint.convert hf2fp8   --load hf/ --out hf_fp8/ [--block 128] [--ue8m0]
    python -m relax_b200.checkpoint.convert fp82bf16 --load hf_fp8/ --out hf_bf16/
    python -m relax_b200.checkpoint.convert hf2int4  --load hf/ --out hf_int4/ [--group 128]
    python -m relax_b200.checkpoint.convert int42bf16 --load hf_int4/ --out hf_bf16/
    python -m relax_b200.checkpoint.convert mergelora --model-name qwen3-8b --load ckpt/ --adapter adapter.pt --out hf/

int4 layout (W4A16, symmetric, groups of ``group`` input channels): ``<name>.weight_packed`` uint8 ``[out, in/2]``
(low nibble = even column, values offset by 8), ``<name>.weight_scale`` ``[out, in/group]``, and the group size in
``config.json`` under ``quantization_config``.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
from typing import Dict

import torch

from ..models.config import get_config
from . import dist_ckpt
from . import hf as H

_KEEP = ("norm", "embed", "lm_head", "router", "gate.weight", "bias")


def _quantisable(name: str, t: torch.Tensor) -> bool:
    return t.dim() == 2 and name.endswith(".weight") and not any(k in name for k in _KEEP)


def _copy_side_files(src: str, dst: str):
    for fn in os.listdir(src):
        if fn.endswith((".json", ".txt", ".model", ".jinja")) and not fn.startswith("model.safetensors") and fn != "config.json":
            shutil.copy(os.path.join(src, fn), os.path.join(dst, fn))


def _load_cfg_json(d: str) -> dict:
    p = os.path.join(d, "config.json")
    return json.load(open(p)) if os.path.exists(p) else {}


def _save_raw(out: str, state: Dict[str, torch.Tensor], config: dict, max_shard_bytes: int = 5 << 30):
    from safetensors.torch import save_file

    os.makedirs(out, exist_ok=True)
    shards, cur, nb = [], {}, 0
    for k, v in state.items():
        b = v.numel() * v.element_size()
        if cur and nb + b > max_shard_bytes:
            shards.append(cur)
            cur, nb = {}, 0
        cur[k] = v.contiguous().cpu()
        nb += b
    if cur:
        shards.append(cur)
    wm = {}
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors" if len(shards) > 1 else "model.safetensors"
        save_file(sh, os.path.join(out, fn), metadata={"format": "pt"})
        wm.update({k: fn for k in sh})
    json.dump({"metadata": {}, "weight_map": wm}, open(os.path.join(out, "model.safetensors.index.json"), "w"), indent=1)
    json.dump(config, open(os.path.join(out, "config.json"), "w"), indent=1)


# ----------------------------------------------------------------------------- int4 (W4A16)
def pack_int4(w: torch.Tensor, group: int):
    out_f, in_f = w.shape
    assert in_f % group == 0 and in_f % 2 == 0
    g = w.float().view(out_f, in_f // group, group)
    scale = g.abs().amax(-1, keepdim=True).clamp_min(1e-8) / 7.0
    q = torch.round(g / scale).clamp(-8, 7).to(torch.int16).view(out_f, in_f) + 8
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8)
    return packed, scale.squeeze(-1).to(w.dtype)


def unpack_int4(packed: torch.Tensor, scale: torch.Tensor, group: int, dtype=torch.bfloat16) -> torch.Tensor:
    out_f = packed.shape[0]
    lo = (packed & 0xF).to(torch.int16) - 8
    hi = (packed >> 4).to(torch.int16) - 8
    q = torch.stack([lo, hi], -1).view(out_f, -1).float()
    return (q.view(out_f, -1, group) * scale.float().unsqueeze(-1)).view(out_f, -1).to(dtype)


# ----------------------------------------------------------------------------- commands
def dist2hf(a):
    cfg = get_config(a.model_name)
    it = dist_ckpt.read_latest_iteration(a.load)
    d = dist_ckpt.iter_dir(a.load, it) if it is not None else a.load
    state = dist_ckpt.load_full_tensors(d)
    hf_state = H.convert_state_to_hf(cfg, {k: v for k, v in state.items() if not k.startswith("optimizer.")})
    H.save_hf_checkpoint(a.out, cfg, hf_state, quantize_fp8=a.fp8, fp8_block=a.block)


def hf2dist(a):
    from ..models.transformer import GPTModel
    from ..parallel.state import single_process_state

    cfg = get_config(a.model_name)
    meg = H.hf_to_megatron_state(cfg, H.load_hf_checkpoint(a.load))
    model = GPTModel(cfg, device="cpu")
    own = dict(model.named_parameters())
    with torch.no_grad():
        for k, v in meg.items():
            own[k].copy_(v)
    dist_ckpt.save_checkpoint(a.out, 0, cfg, single_process_state(), model)


def hf2fp8(a):
    from .. import ops

    st = H.load_hf_checkpoint(a.load, dequantize=True)
    out = {}
    for k, v in st.items():
        if _quantisable(k, v):
            q, s = ops.blockwise_cast_to_fp8(v, a.block, a.ue8m0)
            out[k], out[k + "_scale_inv"] = q, s
        else:
            out[k] = v
    c = _load_cfg_json(a.load)
    c["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [a.block, a.block],
                                "activation_scheme": "dynamic", "scale_fmt": "ue8m0" if a.ue8m0 else "fp32"}
    _save_raw(a.out, out, c)
    _copy_side_files(a.load, a.out)


def fp82bf16(a):
    st = H.load_hf_checkpoint(a.load, dequantize=True, dtype=torch.bfloat16)
    c = _load_cfg_json(a.load)
    c.pop("quantization_config", None)
    _save_raw(a.out, st, c)
    _copy_side_files(a.load, a.out)


def hf2int4(a):
    st = H.load_hf_checkpoint(a.load, dequantize=True)
    out = {}
    for k, v in st.items():
        if _quantisable(k, v) and v.shape[1] % a.group == 0:
            base = k[: -len(".weight")]
            out[base + ".weight_packed"], out[base + ".weight_scale"] = pack_int4(v, a.group)
        else:
            out[k] = v
    c = _load_cfg_json(a.load)
    c["quantization_config"] = {"quant_method": "compressed-tensors", "format": "pack-quantized", "num_bits": 4,
                                "symmetric": True, "group_size": a.group}
    _save_raw(a.out, out, c)
    _copy_side_files(a.load, a.out)


def int42bf16(a):
    st = H.load_hf_checkpoint(a.load, dequantize=False)
    c = _load_cfg_json(a.load)
    group = c.get("quantization_config", {}).get("group_size", 128)
    out = {}
    for k, v in st.items():
        if k.endswith(".weight_packed"):
            base = k[: -len(".weight_packed")]
            out[base + ".weight"] = unpack_int4(v, st[base + ".weight_scale"], group)
        elif not k.endswith(".weight_scale"):
            out[k] = v
    c.pop("quantization_config", None)
    _save_raw(a.out, out, c)
    _copy_side_files(a.load, a.out)


def mergelora(a):
    """Fold an adapter (``<module>.lora_A`` / ``.lora_B`` tensors saved by ``train.lora.adapter_state_dict``) into
    the base weights of a torch-distributed checkpoint and export HF safetensors."""
    cfg = get_config(a.model_name)
    it = dist_ckpt.read_latest_iteration(a.load)
    d = dist_ckpt.iter_dir(a.load, it) if it is not None else a.load
    state = {k: v for k, v in dist_ckpt.load_full_tensors(d).items() if not k.startswith("optimizer.")}
    ad = torch.load(a.adapter, map_location="cpu", weights_only=True)
    scale = a.alpha / a.rank if a.rank else 1.0
    for k in [k for k in ad if k.endswith(".lora_A")]:
        mod = k[: -len(".lora_A")]
        A, B = ad[k].float(), ad[mod + ".lora_B"].float()
        w = state[mod + ".weight"]
        state[mod + ".weight"] = (w.float() + scale * (B @ A)).to(w.dtype)
    H.save_hf_checkpoint(a.out, cfg, H.convert_state_to_hf(cfg, state))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name, fn in [("dist2hf", dist2hf), ("hf2dist", hf2dist), ("hf2fp8", hf2fp8), ("fp82bf16", fp82bf16),
                     ("hf2int4", hf2int4), ("int42bf16", int42bf16), ("mergelora", mergelora)]:
        p = sub.add_parser(name)
        p.set_defaults(fn=fn)
        p.add_argument("--load", required=True)
        p.add_argument("--out", required=True)
        p.add_argument("--model-name", default=None)
        p.add_argument("--block", type=int, default=128)
        p.add_argument("--group", type=int, default=128)
        p.add_argument("--ue8m0", action="store_true")
        p.add_argument("--fp8", action="store_true")
        p.add_argument("--adapter", default=None)
        p.add_argument("--rank", type=int, default=0)
        p.add_argument("--alpha", type=float, default=1.0)
    a = ap.parse_args(argv)
    a.fn(a)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
