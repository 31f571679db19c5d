"""Fused GEMM + collective kernels over NVLink peer memory (2 GPUs), against an fp32 statement of the
same math, and the bounded wait of the peer protocol (1 GPU, a counter that nothing bumps)."""
import os

import pytest
import torch

from tests._mp import run_distributed

pytestmark = pytest.mark.gpu


def _two_gpus():
    return torch.cuda.is_available() and torch.cuda.device_count() >= 2


def _group(world):
    import torch.distributed as dist
    from relax_b200.parallel.state import GroupInfo

    return GroupInfo(group=dist.group.WORLD, ranks=tuple(range(world)), rank=dist.get_rank())


def _inputs(step, rank_of, M, N, K, dev):
    g = torch.Generator(device="cpu").manual_seed(1000 * step + rank_of)
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    return x, w


def _ar_worker(rank, world, shapes, graph):
    from relax_b200.ops import cuda as C
    from relax_b200.parallel.symm_mem import SymmComm

    dev = torch.device("cuda", rank)
    comm = SymmComm(_group(world), dev, workspace_mb=64)
    worst = 0.0
    step = 0
    for (M, N, K) in shapes:
        for rep in range(3):
            step += 1
            g = torch.Generator(device="cpu").manual_seed(7 + step)
            res = torch.randn(M, N, generator=g).to(torch.bfloat16).to(dev)
            nw = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.bfloat16).to(dev)
            x, w = _inputs(step, rank, M, N, K, dev)
            h, y = comm.gemm_ar_add_rmsnorm(x, w, res, nw, 1e-6)
            ref = res.float()
            for r in range(world):
                xr, wr = _inputs(step, r, M, N, K, dev)
                ref = ref + xr.float() @ wr.float().t()
            ref_h = ref.to(torch.bfloat16).float()
            ref_y = ref_h * torch.rsqrt(ref_h.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
            C.check_error_flag(dev)
            worst = max(worst, (h.float() - ref_h).abs().max().item(), (y.float() - ref_y).abs().max().item())
    if graph:
        M, N, K = shapes[0]
        x, w = _inputs(99, rank, M, N, K, dev)
        res = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        s = torch.cuda.Stream(dev)
        with torch.cuda.stream(s):
            comm.gemm_ar_add_rmsnorm(x, w, res, None, 0.0)
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=s):
                h1, _ = comm.gemm_ar_add_rmsnorm(x, w, res, None, 0.0)
                h2, _ = comm.gemm_ar_add_rmsnorm(h1[:, :K].contiguous(), w, res, None, 0.0)
            for _ in range(5):
                gr.replay()
        torch.cuda.synchronize(dev)
        C.check_error_flag(dev)
        ref = sum((_inputs(99, r, M, N, K, dev)[0].float() @ _inputs(99, r, M, N, K, dev)[1].float().t()) for r in range(world))
        worst = max(worst, (h1.float() - ref.to(torch.bfloat16).float()).abs().max().item())
    torch.cuda.synchronize(dev)
    comm.close()
    return worst


@pytest.mark.skipif(not _two_gpus(), reason="needs 2 GPUs")
def test_gemm_allreduce_residual_rmsnorm_two_ranks():
    shapes = [(80, 1024, 512), (16, 4096, 2048), (200, 512, 1536), (1024, 1024, 256)]
    worst = run_distributed(_ar_worker, 2, shapes, True, backend="nccl", timeout=600)
    assert max(worst) < 0.08, worst


def _rs_worker(rank, world, shapes):
    from relax_b200.ops import cuda as C
    from relax_b200.parallel.symm_mem import SymmComm

    dev = torch.device("cuda", rank)
    comm = SymmComm(_group(world), dev, workspace_mb=64)
    worst = 0.0
    step = 100
    for (M, N, K, kn) in shapes:
        for rep in range(2):
            step += 1
            x, w = _inputs(step, rank, M, N, K, dev)
            wk = w.t().contiguous() if kn else w
            y = comm.gemm_rs(x, wk, w_is_kn=kn)
            ref = 0
            for r in range(world):
                xr, wr = _inputs(step, r, M, N, K, dev)
                ref = ref + xr.float() @ wr.float().t()
            rows = M // world
            ref = ref[rank * rows:(rank + 1) * rows]
            C.check_error_flag(dev)
            worst = max(worst, (y.float() - ref).abs().max().item() / max(1.0, ref.abs().max().item()))
    torch.cuda.synchronize(dev)
    comm.close()
    return worst


@pytest.mark.skipif(not _two_gpus(), reason="needs 2 GPUs")
def test_gemm_reduce_scatter_two_ranks():
    shapes = [(512, 1024, 512, False), (2048, 512, 1024, False), (1024, 768, 512, True)]
    worst = run_distributed(_rs_worker, 2, shapes, backend="nccl", timeout=600)
    assert max(worst) < 0.02, worst


def _ag_worker(rank, world, shapes):
    from relax_b200.ops import cuda as C
    from relax_b200.parallel.symm_mem import SymmComm

    dev = torch.device("cuda", rank)
    comm = SymmComm(_group(world), dev, workspace_mb=64)
    worst = 0.0
    step = 200
    for (Ts, N, K) in shapes:
        for rep in range(3):
            step += 1
            x, _ = _inputs(step, rank, Ts, 8, K, dev)
            _, w = _inputs(step, 77, 8, N, K, dev)   # same weight shard on both ranks: checks rows only
            y, _ = comm.ag_gemm(x, w)
            xs = [_inputs(step, r, Ts, 8, K, dev)[0] for r in range(world)]
            ref = torch.cat(xs).float() @ w.float().t()
            C.check_error_flag(dev)
            worst = max(worst, (y.float() - ref).abs().max().item() / max(1.0, ref.abs().max().item()))
    torch.cuda.synchronize(dev)
    comm.close()
    return worst


@pytest.mark.skipif(not _two_gpus(), reason="needs 2 GPUs")
def test_allgather_gemm_two_ranks():
    shapes = [(128, 256, 256), (512, 1024, 512), (1280, 768, 1024)]
    worst = run_distributed(_ag_worker, 2, shapes, backend="nccl", timeout=600)
    assert max(worst) < 0.02, worst


def test_peer_wait_runs_out_and_reports():
    """A claimed second rank that never launches: the wait for its arrivals expires, the kernel sets the error
    flag and returns, and the context stays usable."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from relax_b200.ops import cuda as C

    dev = torch.device("cuda", 0)
    _C = C._load()
    ws0 = _C.symm_alloc(8 << 20, 0)
    ws1 = _C.symm_alloc(8 << 20, 0)
    sg0 = _C.symm_alloc(1024, 0)
    sg1 = _C.symm_alloc(1024, 0)
    try:
        M, N, K = 32, 256, 256
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w = torch.randn(N, K, device=dev).to(torch.bfloat16)
        state = torch.zeros(8, dtype=torch.int32, device=dev)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        err = C.err_flag(dev)
        _C.gemm_ar_rmsnorm(x, w, [ws0, ws1], [sg0, sg1], 0, state, None, None, out, None, 0.0, 1, 64, False, False,
                           200_000_000, err)
        torch.cuda.synchronize(dev)
        assert int(err.item()) == 3
        err.zero_()
        # the context still works
        y = C.matmul_nt(x, w)
        torch.testing.assert_close(y.float(), x.float() @ w.float().t(), atol=0.5, rtol=0.05)
    finally:
        for p in (ws0, ws1, sg0, sg1):
            _C.symm_free(p, 0)


def _dpopt_worker(rank, world):
    """Two data-parallel ranks: the fused optimizer step (peer loads / stores) against the NCCL statement."""
    import dataclasses

    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel
    from relax_b200.ops import cuda as C
    from relax_b200.parallel.state import ParallelDims, init_parallel_state
    from relax_b200.train.optimizer import DistributedOptimizer, OptimizerConfig

    dev = torch.device("cuda", rank)
    ps = init_parallel_state(ParallelDims(dp=2))
    cfg = get_config("qwen3-0.6b", num_layers=2, vocab_size=2048)
    outs = []
    for fused in (True, False):
        torch.manual_seed(0)
        model = GPTModel(cfg, ps, device=dev, seed=0)
        opt = DistributedOptimizer(model, ps, OptimizerConfig(lr=1e-3, clip_grad=1.0, weight_decay=0.01, fused_dp=fused))
        assert (opt._symm is not None) == fused
        for step in range(3):
            opt.zero_grad()
            g = torch.Generator(device="cpu").manual_seed(100 * step + rank)
            for p in opt.params:
                p.main_grad.copy_((torch.randn(p.shape, generator=g) * 0.01).to(dev))
            norm, skipped = opt.step()
            assert not skipped
        torch.cuda.synchronize(dev)
        C.check_error_flag(dev)
        outs.append((opt.param_buf.float().clone(), float(norm)))
    (pf, nf), (pn, nn) = outs
    return float((pf - pn).abs().max()), abs(nf - nn) / max(nn, 1e-9), float(pf.abs().sum())


def _dpopt_sleep_worker(rank, world):
    """Step, offload (sleep), onload (wake up), step on different gradients: the fused path must reduce the NEW
    gradients, i.e. keep accumulating into the symmetric buffer its reduce kernel reads."""
    from relax_b200.models.config import get_config
    from relax_b200.models.transformer import GPTModel
    from relax_b200.ops import cuda as C
    from relax_b200.parallel.state import ParallelDims, init_parallel_state
    from relax_b200.train.optimizer import DistributedOptimizer, OptimizerConfig

    dev = torch.device("cuda", rank)
    ps = init_parallel_state(ParallelDims(dp=2))
    cfg = get_config("qwen3-0.6b", num_layers=2, vocab_size=2048)
    outs = []
    for fused in (True, False):
        model = GPTModel(cfg, ps, device=dev, seed=0)
        opt = DistributedOptimizer(model, ps, OptimizerConfig(lr=1e-3, clip_grad=1.0, fused_dp=fused))
        norms = []
        for step in range(3):
            opt.zero_grad()
            g = torch.Generator(device="cpu").manual_seed(100 * step + rank)
            for p in opt.params:
                p.main_grad.copy_((torch.randn(p.shape, generator=g) * 0.01 * (step + 1)).to(dev))
            norm, skipped = opt.step()
            norms.append(float(norm))
            assert not skipped
            opt.offload_state()
            if fused:
                assert opt.grad_buf is not None and opt.grad_buf.data_ptr() == opt._symm["grad"].local_ptr
            opt.onload_state()
            if fused:
                assert opt.params[0].main_grad.data_ptr() >= opt._symm["grad"].local_ptr
        torch.cuda.synchronize(dev)
        C.check_error_flag(dev)
        master = opt.master_shard_fp32().clone()
        outs.append((opt.param_buf.float().clone(), norms, master))
        opt.close()
    (pf, nf, mf), (pn, nn, mn) = outs
    nrel = max(abs(a - b) / max(b, 1e-9) for a, b in zip(nf, nn))
    return float((pf - pn).abs().max()), nrel, float((mf - mn).abs().max()), nn


@pytest.mark.skipif(not _two_gpus(), reason="needs 2 GPUs")
def test_fused_distributed_optimizer_survives_sleep_and_wake_up():
    out = run_distributed(_dpopt_sleep_worker, 2, backend="nccl", timeout=600)
    for diff, nrel, mdiff, norms in out:
        assert norms[0] != norms[1] != norms[2]          # every step saw its own gradients
        assert diff <= 5e-4 and nrel < 1e-4 and mdiff <= 1e-6, out


@pytest.mark.skipif(not _two_gpus(), reason="needs 2 GPUs")
def test_fused_distributed_optimizer_matches_nccl_path():
    out = run_distributed(_dpopt_worker, 2, backend="nccl", timeout=600)
    for diff, nrel, mass in out:
        # the two paths round the clip factor differently in the last bit: allow one bf16 ulp at |w| < 0.06
        assert diff <= 5e-4 and nrel < 1e-4 and mass > 0, out
    assert out[0][2] == out[1][2]      # both ranks hold the same parameters after the fused all-gather


def _cp_worker(rank, world, L, valid):
    """Zig-zag context parallelism with in-kernel KV reads from the peer, against full attention on one GPU."""
    from relax_b200 import ops
    from relax_b200.ops import cuda as C
    from relax_b200.parallel.cp_peer import CPComm, peer_attention

    dev = torch.device("cuda", rank)
    Hq, Hkv, D, cp = 8, 2, 128, world
    cs = L // (2 * cp)
    g = torch.Generator().manual_seed(5)
    qf = (torch.randn(L, Hq, D, generator=g) * 0.5).bfloat16().to(dev)
    kf = (torch.randn(L, Hkv, D, generator=g) * 0.5).bfloat16().to(dev)
    vf = (torch.randn(L, Hkv, D, generator=g) * 0.5).bfloat16().to(dev)
    dof = (torch.randn(L, Hq, D, generator=g) * 0.1).bfloat16().to(dev)
    idx = torch.cat([torch.arange(rank * cs, (rank + 1) * cs), torch.arange((2 * cp - 1 - rank) * cs, (2 * cp - rank) * cs)]).to(dev)
    comm = CPComm(_group(world), dev, 2 * cs, Hq, Hkv)
    worst = 0.0
    for rep in range(2):
        # reference: the whole (valid) sequence on this GPU
        qr, kr, vr = (t[:valid].clone().requires_grad_() for t in (qf, kf, vf))
        cu = torch.tensor([0, valid], dtype=torch.int32, device=dev)
        o_ref = ops.attention_varlen(qr, kr, vr, cu, causal=True)
        o_ref.backward(dof[:valid])
        pad = lambda t: torch.cat([t, torch.zeros(L - valid, *t.shape[1:], dtype=t.dtype, device=dev)])
        q, k, v = (t[idx].clone().requires_grad_() for t in (qf, kf, vf))
        o = peer_attention(q, k, v, comm, valid)
        o.backward(dof[idx])
        torch.cuda.synchronize(dev)
        C.check_error_flag(dev)
        live = idx < valid
        for got, ref in ((o, pad(o_ref.detach())[idx]), (q.grad, pad(qr.grad)[idx]), (k.grad, pad(kr.grad)[idx]),
                         (v.grad, pad(vr.grad)[idx])):
            worst = max(worst, float((got.float() - ref.float())[live].abs().max()))
    comm.close()
    return worst


@pytest.mark.skipif(not _two_gpus(), reason="needs 2 GPUs")
@pytest.mark.parametrize("L,valid", [(1024, 1024), (1024, 900)])
def test_context_parallel_attention_reads_peer_kv(L, valid):
    worst = run_distributed(_cp_worker, 2, L, valid, backend="nccl", timeout=600)
    assert max(worst) < 0.03, worst


def _ep_worker(rank, world):
    """Variable-size token exchange by peer stores against all_to_all_single, forward and backward."""
    import torch.distributed as dist

    from relax_b200.ops import cuda as C
    from relax_b200.parallel.ep_peer import EPComm, peer_all_to_all

    dev = torch.device("cuda", rank)
    H, E = 256, 8
    comm = EPComm(_group(world), dev, capacity_rows=4096, hidden=H)
    worst = 0.0
    for rep in range(3):
        g = torch.Generator().manual_seed(31 * rep + rank)
        counts = torch.randint(0, 40, (E,), generator=g).to(dev)
        allc = comm.exchange_counts(counts)
        ref = [torch.empty_like(counts) for _ in range(world)]
        dist.all_gather(ref, counts)
        assert torch.equal(allc, torch.stack(ref))
        el = E // world
        matrix = allc.view(world, world, el).sum(-1).tolist()
        n_send = int(counts.sum())
        x = torch.randn(n_send, H, generator=g).bfloat16().to(dev).requires_grad_()
        y = peer_all_to_all(x, matrix, comm)
        in_splits, out_splits = matrix[rank], [matrix[s][rank] for s in range(world)]
        y_ref = torch.empty(sum(out_splits), H, dtype=x.dtype, device=dev)
        dist.all_to_all_single(y_ref, x.detach().contiguous(), out_splits, in_splits)
        gy = torch.randn(y.shape, generator=g).bfloat16().to(dev)
        y.backward(gy)
        gx_ref = torch.empty(n_send, H, dtype=x.dtype, device=dev)
        dist.all_to_all_single(gx_ref, gy.contiguous(), in_splits, out_splits)
        torch.cuda.synchronize(dev)
        C.check_error_flag(dev)
        worst = max(worst, float((y.float() - y_ref.float()).abs().max()) if y.numel() else 0.0,
                    float((x.grad.float() - gx_ref.float()).abs().max()))
    comm.close()
    return worst


@pytest.mark.skipif(not _two_gpus(), reason="needs 2 GPUs")
def test_expert_parallel_exchange_by_peer_stores():
    assert max(run_distributed(_ep_worker, 2, backend="nccl", timeout=600)) == 0.0
