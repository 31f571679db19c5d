import copy

import torch

from relax_b200.models.config import get_config
from relax_b200.models.transformer import GPTModel
from relax_b200.train.optimizer import DistributedOptimizer, OptimizerConfig, _join_fp32, _split_fp32, lr_at
from relax_b200.parallel.state import single_process_state
from tests._mp import run_distributed


def test_split_master_is_exact():
    torch.manual_seed(0)
    x = torch.randn(10000) * torch.logspace(-6, 3, 10000)
    hi, rem = _split_fp32(x, torch.bfloat16)
    # the 16-bit value is a nearest bf16 neighbour (exact ties may round either way) ...
    assert (hi.float() - x).abs().le((x.to(torch.bfloat16).float() - x).abs()).all()
    assert torch.equal(_join_fp32(hi, rem), x)              # ... and the fp32 master is recovered bit-exactly
    tie = torch.tensor([0x3F808000, 0x3F818000, -0x407F8000 + 2**32 - 2**32], dtype=torch.int32).view(torch.float32)
    h2, r2 = _split_fp32(tie, torch.bfloat16)
    assert torch.equal(_join_fp32(h2, r2), tie)


def test_lr_schedule():
    c = OptimizerConfig(lr=1.0, min_lr=0.1, lr_warmup_iters=2, lr_decay_iters=12, lr_decay_style="cosine")
    assert lr_at(c, 0) == 0.5 and lr_at(c, 1) == 1.0
    assert abs(lr_at(c, 7) - 0.55) < 1e-6 and abs(lr_at(c, 100) - 0.1) < 1e-9
    c.lr_decay_style = "linear"
    assert abs(lr_at(c, 7) - 0.55) < 1e-6
    assert lr_at(OptimizerConfig(lr=3e-4), 1234) == 3e-4


def _adamw_reference(model, steps_grads, cfg):
    ps = [p.detach().clone().float() for p in model.parameters()]
    opt = torch.optim.AdamW(ps, lr=cfg.lr, betas=(cfg.adam_beta1, cfg.adam_beta2), eps=cfg.adam_eps,
                            weight_decay=cfg.weight_decay)
    for grads in steps_grads:
        tot = torch.sqrt(sum(g.float().pow(2).sum() for g in grads))
        clip = min(1.0, cfg.clip_grad / (tot + 1e-6)) if cfg.clip_grad > 0 else 1.0
        for p, g in zip(ps, grads):
            p.grad = g.float() * clip
        opt.step()
    return ps


def test_single_rank_matches_torch_adamw_fp32():
    cfg = get_config("tiny")
    m = GPTModel(cfg, seed=0)
    ocfg = OptimizerConfig(lr=1e-3, weight_decay=0.01, clip_grad=1.0)
    ref_model = copy.deepcopy(m)
    opt = DistributedOptimizer(m, single_process_state(), ocfg)
    torch.manual_seed(0)
    all_grads = []
    for _ in range(3):
        grads = [torch.randn_like(p) * 0.01 for p in opt.params]
        all_grads.append(grads)
        opt.zero_grad()
        for p, g in zip(opt.params, grads):
            p.main_grad.add_(g)
        norm, skipped = opt.step()
        assert not skipped and norm > 0
    # reference in the optimizer's parameter order
    name_of = {id(p): n for n, p in m.named_parameters()}
    ref_params = dict(ref_model.named_parameters())

    class _M:
        def parameters(self_inner):
            return [ref_params[name_of[id(p)]] for p in opt.params]

    exp = _adamw_reference(_M(), all_grads, ocfg)
    for p, e in zip(opt.params, exp):
        assert torch.allclose(p.data, e, atol=1e-6), (p.data - e).abs().max()


def test_bf16_split_master_tracks_fp32_master():
    cfg = get_config("tiny", dtype="bf16")
    m = GPTModel(cfg, seed=0)
    opt = DistributedOptimizer(m, single_process_state(), OptimizerConfig(lr=1e-4, clip_grad=0))
    assert opt.split_master and opt.master is None
    master0 = opt.master_shard_fp32().clone()
    assert torch.equal(master0, opt.param_buf.float())
    torch.manual_seed(0)
    g = torch.randn(opt.total) * 1e-3
    ref = master0.clone()
    mm, vv = torch.zeros_like(ref), torch.zeros_like(ref)
    from relax_b200.ops.reference import adam_step
    for step in range(1, 4):
        opt.zero_grad()
        opt.grad_buf.add_(g)
        opt.step()
        adam_step(ref, g, mm, vv, step, 1e-4, 0.9, 0.999, 1e-8, 0.0)
        assert torch.equal(opt.master_shard_fp32(), ref)     # tiny updates are not lost to bf16 rounding
        assert (opt.param_buf.float() - ref).abs().le((ref.to(torch.bfloat16).float() - ref).abs()).all()


def _dp_worker(rank, world):
    from relax_b200.parallel.state import ParallelDims, init_parallel_state

    cfg = get_config("tiny")
    ps = init_parallel_state(ParallelDims(dp=2))
    m = GPTModel(cfg, ps, seed=0)
    ocfg = OptimizerConfig(lr=1e-3, clip_grad=1.0)
    opt = DistributedOptimizer(m, ps, ocfg)
    single = GPTModel(cfg, single_process_state(), seed=0)
    sopt = DistributedOptimizer(single, single_process_state(), ocfg)
    for step in range(2):
        gs = []
        for r in range(world):
            torch.manual_seed(100 * step + r)
            gs.append(torch.randn(opt.total) * 0.01)
        opt.zero_grad()
        opt.grad_buf.add_(gs[rank])
        n1, _ = opt.step()
        sopt.zero_grad()
        sopt.grad_buf[: opt.total].add_((gs[0] + gs[1])[: sopt.total] / 2)
        n2, _ = sopt.step()
    # padding differs between layouts; compare parameter by parameter
    for (n, p), (_, q) in zip(m.named_parameters(), single.named_parameters()):
        assert torch.allclose(p, q, atol=1e-6), n
    sd = opt.state_dict()
    opt.load_state_dict(sd)
    return True


def test_dp2_equals_single_rank_average():
    assert all(run_distributed(_dp_worker, 2))
