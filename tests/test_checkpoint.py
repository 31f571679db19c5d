"""Checkpoint round trips: DCP-format sharded checkpoints across parallel layouts, HF safetensors
both ways, rotation and resume bookkeeping."""
import os

import pytest
import torch

from relax_b200.checkpoint import dist_ckpt as D
from relax_b200.checkpoint import hf as HF
from relax_b200.models.config import get_config
from relax_b200.models.transformer import GPTModel
from relax_b200.parallel.state import single_process_state
from relax_b200.train.optimizer import DistributedOptimizer, OptimizerConfig
from tests._mp import run_distributed


def _randomise(model, seed):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * 0.05)


def test_hf_round_trip_and_safetensors(tmp_path):
    for name in ("tiny", "tiny-moe"):
        cfg = get_config(name)
        m = GPTModel(cfg, seed=1)
        _randomise(m, 3)
        state = {k: v.detach() for k, v in m.named_parameters()}
        hf = HF.convert_state_to_hf(cfg, state)
        assert "model.layers.0.self_attn.q_proj.weight" in hf and "model.layers.1.self_attn.k_norm.weight" in hf
        if cfg.is_moe:
            assert hf["model.layers.0.mlp.experts.7.down_proj.weight"].shape == (cfg.hidden_size, cfg.moe_ffn_hidden_size)
        else:
            assert hf["model.layers.0.mlp.gate_proj.weight"].shape == (cfg.ffn_hidden_size, cfg.hidden_size)
        back = HF.hf_to_megatron_state(cfg, hf)
        for k, v in state.items():
            assert torch.equal(back[k], v), k
        d = str(tmp_path / name)
        HF.save_hf_checkpoint(d, cfg, hf, max_shard_bytes=1 << 20)
        assert HF.is_hf_checkpoint(d) and len([f for f in os.listdir(d) if f.endswith(".safetensors")]) > 1
        loaded = HF.load_hf_checkpoint(d)
        for k, v in hf.items():
            assert torch.equal(loaded[k], v), k


def test_hf_fp8_export_dequantises_close(tmp_path):
    cfg = get_config("tiny", dtype="bf16")
    m = GPTModel(cfg, seed=2)
    hf = HF.convert_state_to_hf(cfg, {k: v.detach() for k, v in m.named_parameters()})
    d = str(tmp_path / "fp8")
    HF.save_hf_checkpoint(d, cfg, hf, quantize_fp8=True, fp8_block=64)
    raw = HF.load_hf_checkpoint(d, dequantize=False)
    assert raw["model.layers.0.mlp.down_proj.weight"].dtype == torch.float8_e4m3fn
    assert "model.layers.0.mlp.down_proj.weight_scale_inv" in raw and raw["model.norm.weight"].dtype == torch.bfloat16
    deq = HF.load_hf_checkpoint(d)
    w, r = hf["model.layers.0.mlp.down_proj.weight"].float(), deq["model.layers.0.mlp.down_proj.weight"].float()
    assert (w - r).abs().max() <= 0.07 * w.abs().max()


def _save_tp2(rank, world, save):
    from relax_b200.parallel.state import ParallelDims, init_parallel_state

    cfg = get_config("tiny")
    ps = init_parallel_state(ParallelDims(tp=2))
    m = GPTModel(cfg, ps, seed=5)
    opt = DistributedOptimizer(m, ps, OptimizerConfig(lr=1e-3))
    opt.zero_grad()
    opt.grad_buf.add_(0.01)
    opt.step()
    D.save_checkpoint(save, 7, cfg, ps, m, opt, extra={"rollout_id": 7})
    # same layout: everything, optimizer included, comes back
    m2 = GPTModel(cfg, ps, seed=99)
    opt2 = DistributedOptimizer(m2, ps, OptimizerConfig(lr=1e-3))
    common = D.load_checkpoint(save, cfg, ps, m2, opt2)
    assert common["rollout_id"] == 7 and opt2.step_count == 1
    for (n, a), (_, b) in zip(m.named_parameters(), m2.named_parameters()):
        assert torch.equal(a, b), n
    assert torch.equal(opt.exp_avg, opt2.exp_avg) and torch.equal(opt.master_shard_fp32(), opt2.master_shard_fp32())
    return {n: p.detach().clone() for n, p in m.named_parameters()}


def test_dist_checkpoint_resharding_tp2_to_tp1(tmp_path):
    save = str(tmp_path / "ckpt")
    shards = run_distributed(_save_tp2, 2, save)
    assert D.read_latest_iteration(save) == 7 and D.is_dist_checkpoint(save)
    assert D.resolve_start_rollout_id(save) == 8 and D.resolve_start_rollout_id(save, 3) == 3
    cfg = get_config("tiny")
    ps = single_process_state()
    m = GPTModel(cfg, ps, seed=123)
    D.load_checkpoint(save, cfg, ps, m)
    # the TP1 model equals the concatenation of the TP2 shards
    full = dict(m.named_parameters())
    q = "decoder.layers.0.self_attention.linear_qkv.weight"
    assert torch.equal(full[q], torch.cat([shards[0][q], shards[1][q]], 0))
    o = "decoder.layers.1.self_attention.linear_proj.weight"
    assert torch.equal(full[o], torch.cat([shards[0][o], shards[1][o]], 1))
    f1 = "decoder.layers.0.mlp.linear_fc1.weight"
    F = cfg.ffn_hidden_size // 2
    exp = torch.cat([shards[0][f1][:F], shards[1][f1][:F], shards[0][f1][F:], shards[1][f1][F:]], 0)
    assert torch.equal(full[f1], exp)
    # the index is a genuine torch.distributed.checkpoint Metadata object: DCP itself can read the files
    import torch.distributed.checkpoint as dcp

    sd = {q: torch.zeros_like(full[q])}
    dcp.load(sd, checkpoint_id=D.iter_dir(save, 7), no_dist=True)
    assert torch.equal(sd[q], full[q])
    all_t = D.load_full_tensors(D.iter_dir(save, 7), names={q})
    assert torch.equal(all_t[q], full[q])


def test_rotation_keeps_newest(tmp_path):
    save = str(tmp_path)
    for it in (1, 2, 3, 10):
        os.makedirs(D.iter_dir(save, it))
    assert D.rotate_checkpoints(save, 2) == [1, 2]
    assert sorted(os.listdir(save)) == ["iter_0000003", "iter_0000010"]
    assert D.rotate_checkpoints(save, None) == []


def _hf_tp_worker(rank, world, path):
    import torch
    from relax_b200.checkpoint import hf as H
    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel
    from relax_b200.parallel.state import ParallelDims, init_parallel_state

    ps = init_parallel_state(ParallelDims(tp=2))
    cfg = get_config("tiny")
    m = GPTModel(cfg, ps, seed=99)                 # different init: everything must come from the files
    assert H.load_hf_into_model(path, cfg, ps, m) == []
    toks = torch.arange(8) + 3
    h = m(toks, torch.arange(8), torch.tensor([0, 8], dtype=torch.int32))
    lp, _ = m.log_probs(h[:-1], toks[1:], with_entropy=False)
    return lp.detach()


def test_hf_checkpoint_loads_into_tp2_and_controller_flags(tmp_path):
    import torch
    from relax_b200.checkpoint import hf as H
    from relax_b200.config.arguments import parse_args
    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel
    from relax_b200.orchestration.controller import Controller
    from tests._mp import run_distributed

    cfg = get_config("tiny")
    src = GPTModel(cfg, seed=5)
    d = str(tmp_path / "hf")
    H.save_hf_checkpoint(d, cfg, H.convert_state_to_hf(cfg, {k: v.detach() for k, v in src.named_parameters()}))
    toks = torch.arange(8) + 3
    h = src(toks, torch.arange(8), torch.tensor([0, 8], dtype=torch.int32))
    ref, _ = src.log_probs(h[:-1], toks[1:], with_entropy=False)
    for lp in run_distributed(_hf_tp_worker, 2, d):
        assert torch.allclose(lp, ref.detach(), atol=1e-5)
    # the controller: --hf-checkpoint initialises policy, rollout weights and reference; --save-hf exports after a step
    out = tmp_path / "ckpt"
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2",
                    "--global-batch-size", "4", "--num-rollout", "1", "--rollout-max-response-len", "8", "--hf-checkpoint", d,
                    "--save", str(out), "--save-interval", "1", "--save-hf", str(tmp_path / "export")])
    c = Controller(a, device="cpu")
    got = dict(c.runner.actor.model.named_parameters())
    for k, v in src.named_parameters():
        assert torch.equal(got[k].detach(), v.detach()), k
    assert torch.equal(c.runner.engine.weights.p["final_norm"], src.decoder.final_layernorm.weight.detach())
    c.training_loop()
    exported = [p for p in (tmp_path / "export").iterdir()]
    assert exported and H.is_hf_checkpoint(str(exported[0]))
    back = H.hf_to_megatron_state(cfg, H.load_hf_checkpoint(str(exported[0])))
    assert set(back) == {k for k, _ in src.named_parameters()}


def test_model_flags_are_checked_against_the_hf_config(tmp_path):
    """A model shape that differs from the ``config.json`` under ``--hf-checkpoint`` is refused with the list of
    differing fields; the matching one passes."""
    import pytest

    for name in ("tiny", "tiny-moe"):
        cfg = get_config(name)
        m = GPTModel(cfg, seed=1)
        d = str(tmp_path / name)
        HF.save_hf_checkpoint(d, cfg, HF.convert_state_to_hf(cfg, {k: v.detach() for k, v in m.named_parameters()}))
        HF.validate_against_hf(cfg, d)
        with pytest.raises(ValueError, match="rope_theta.*|num_layers.*"):
            HF.validate_against_hf(get_config(name, num_layers=cfg.num_layers + 1, rope_theta=5e5), d)
    HF.validate_against_hf(get_config("tiny"), str(tmp_path / "no-such-dir"))        # nothing to compare with: no error
