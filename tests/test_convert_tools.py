"""Checkpoint conversion CLI: dist <-> HF, fp8 and int4 round trips, LoRA merge (tiny model, CPU)."""
import json
import os

import torch

from relax_b200.checkpoint import convert as CV
from relax_b200.checkpoint import dist_ckpt
from relax_b200.checkpoint import hf as H
from relax_b200.models.config import get_config
from relax_b200.models.transformer import GPTModel
from relax_b200.parallel.state import single_process_state


def _save_tiny(tmp_path):
    cfg = get_config("tiny")
    model = GPTModel(cfg, device="cpu", seed=3)
    d = str(tmp_path / "dist")
    dist_ckpt.save_checkpoint(d, 4, cfg, single_process_state(), model)
    return cfg, model, d


def test_dist_to_hf_and_back(tmp_path):
    cfg, model, d = _save_tiny(tmp_path)
    hf_dir, back = str(tmp_path / "hf"), str(tmp_path / "back")
    assert CV.main(["dist2hf", "--model-name", "tiny", "--load", d, "--out", hf_dir]) == 0
    assert H.is_hf_checkpoint(hf_dir)
    assert CV.main(["hf2dist", "--model-name", "tiny", "--load", hf_dir, "--out", back]) == 0
    m2 = GPTModel(cfg, device="cpu", seed=99)
    dist_ckpt.load_checkpoint(back, cfg, single_process_state(), m2)
    for (n, a), (_, b) in zip(model.named_parameters(), m2.named_parameters()):
        assert torch.equal(a, b), n


def test_fp8_and_int4_roundtrips(tmp_path):
    cfg, model, d = _save_tiny(tmp_path)
    hf_dir = str(tmp_path / "hf")
    CV.main(["dist2hf", "--model-name", "tiny", "--load", d, "--out", hf_dir])
    ref = H.load_hf_checkpoint(hf_dir)
    f8, b16 = str(tmp_path / "f8"), str(tmp_path / "b16")
    CV.main(["hf2fp8", "--load", hf_dir, "--out", f8, "--block", "64"])
    raw = H.load_hf_checkpoint(f8, dequantize=False)
    qk = [k for k in raw if k.endswith("_scale_inv")]
    assert qk and raw[qk[0][:-len("_scale_inv")]].dtype == torch.float8_e4m3fn
    assert json.load(open(os.path.join(f8, "config.json")))["quantization_config"]["weight_block_size"] == [64, 64]
    CV.main(["fp82bf16", "--load", f8, "--out", b16])
    deq = H.load_hf_checkpoint(b16)
    assert set(deq) == set(ref)
    for k in ref:
        err = (deq[k].float() - ref[k].float()).abs().max() / ref[k].float().abs().max().clamp_min(1e-6)
        assert err < (0.08 if k + "_scale_inv" in raw else 0.01), (k, float(err))
    i4, b16b = str(tmp_path / "i4"), str(tmp_path / "b16b")
    CV.main(["hf2int4", "--load", hf_dir, "--out", i4, "--group", "32"])
    raw4 = H.load_hf_checkpoint(i4, dequantize=False)
    assert any(k.endswith(".weight_packed") and v.dtype == torch.uint8 for k, v in raw4.items())
    CV.main(["int42bf16", "--load", i4, "--out", b16b])
    deq4 = H.load_hf_checkpoint(b16b)
    assert set(deq4) == set(ref)
    w = torch.randn(8, 64)
    p, s = CV.pack_int4(w, 32)
    assert (CV.unpack_int4(p, s, 32, torch.float32) - w).abs().max() <= s.float().max() * 0.51


def test_merge_lora_cli(tmp_path):
    from relax_b200.train import lora as LR

    cfg, model, d = _save_tiny(tmp_path)
    LR.apply_lora(model, LR.LoRAConfig(rank=4, alpha=8))
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("lora_B"):
                p.normal_(0, 0.05)
    ad = str(tmp_path / "adapter.pt")
    torch.save(LR.adapter_state_dict(model), ad)
    out = str(tmp_path / "merged")
    CV.main(["mergelora", "--model-name", "tiny", "--load", d, "--adapter", ad, "--rank", "4", "--alpha", "8", "--out", out])
    merged_hf = H.load_hf_checkpoint(out)
    want = H.convert_state_to_hf(cfg, dict(LR.merged_named_params(model)))
    for k in want:
        assert torch.allclose(merged_hf[k].float(), want[k].float(), atol=1e-5), k
