"""A/B benchmark of the fused GEMM + collective kernels against the NCCL statements they replace.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m relax_b200.parallel.bench_fused_comm [--timeline]

One process per GPU of one node.  For every shape it times (CUDA events, max over ranks, after warm-up)
the fused kernel, the unfused pair ``GEMM -> NCCL collective (-> add + RMSNorm)`` and the GEMM alone;
the gap between the last two is what a perfect overlap could save.  Decode shapes run inside a CUDA
graph of 20 calls (as the rollout engine runs them); training shapes run eagerly.  ``--timeline``
prints the per-CTA phase stamps of the all-reduce kernel (global timer, microseconds from the first
CTA's start).
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def _time(fn, iters, graph, dev):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=s):
                for _ in range(iters):
                    fn()
            gr.replay()
            torch.cuda.synchronize()
            dist.barrier()
            e0.record(s)
            gr.replay()
            gr.replay()
            e1.record(s)
            torch.cuda.synchronize()
        t = e0.elapsed_time(e1) / (2 * iters)
    else:
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) / iters
    tt = torch.tensor([t], device=dev)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    return tt.item() * 1000   # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--timeline", action="store_true")
    args = ap.parse_args()
    from .. import ops
    from ..ops import cuda as C
    from .state import GroupInfo
    from .symm_mem import SymmComm

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    comm = SymmComm(GroupInfo(dist.group.WORLD, tuple(range(world)), rank), dev, workspace_mb=512)
    say = print if rank == 0 else (lambda *a, **k: None)
    H, F = 4096, 12288

    say(f"== decode: GEMM + all-reduce + residual + RMSNorm, TP{world} (us per call, CUDA graph of 20)")
    for (M, K) in [(16, H // world), (64, H // world), (128, H // world), (64, F // world), (128, F // world), (256, F // world)]:
        x = torch.randn(M, K, device=dev).bfloat16()
        w = (torch.randn(H, K, device=dev) * 0.02).bfloat16()
        res = torch.randn(M, H, device=dev).bfloat16()
        nw = torch.ones(H, device=dev).bfloat16()

        def nccl():
            a = ops.linear(x, w)
            dist.all_reduce(a)
            return ops.add_rmsnorm(a, res, nw, 1e-6)

        tf = _time(lambda: comm.gemm_ar_add_rmsnorm(x, w, res, nw, 1e-6), 20, True, dev)
        tn = _time(nccl, 20, True, dev)
        tl = _time(lambda: ops.add_rmsnorm(ops.linear(x, w), res, nw, 1e-6), 20, True, dev)
        say(f"  M={M:4d} K={K:5d} N={H}: fused {tf:6.1f}   GEMM+NCCL+norm {tn:6.1f}   (no collective {tl:6.1f})")

    say(f"== training: GEMM + reduce-scatter, TP{world} (us per call)")
    for (M, K) in [(5120, H // world), (5120, F // world), (8192, F // world)]:
        x = torch.randn(M, K, device=dev).bfloat16()
        w = (torch.randn(H, K, device=dev) * 0.02).bfloat16()

        def nccl():
            a = ops.linear(x, w)
            out = torch.empty(M // world, H, device=dev, dtype=a.dtype)
            dist.reduce_scatter_tensor(out, a)
            return out

        tf, tn, tl = (_time(f, 5, False, dev) for f in (lambda: comm.gemm_rs(x, w), nccl, lambda: ops.linear(x, w)))
        say(f"  M={M:5d} K={K:5d} N={H}: fused {tf:6.1f}   GEMM+NCCL {tn:6.1f}   (GEMM alone {tl:6.1f})")

    say(f"== training: all-gather + GEMM, TP{world} (us per call)")
    for (Ts, N) in [(5120 // world, 3 * H // world), (5120 // world, 2 * F // world), (8192 // world, 2 * F // world)]:
        x = torch.randn(Ts, H, device=dev).bfloat16()
        w = (torch.randn(N, H, device=dev) * 0.02).bfloat16()
        xfull = torch.randn(Ts * world, H, device=dev).bfloat16()

        def nccl():
            xf = torch.empty(Ts * world, H, device=dev, dtype=x.dtype)
            dist.all_gather_into_tensor(xf, x)
            return ops.linear(xf, w)

        tf, tn, tl = (_time(f, 5, False, dev) for f in (lambda: comm.ag_gemm(x, w), nccl, lambda: ops.linear(xfull, w)))
        say(f"  rows/rank={Ts:5d} N={N:5d} K={H}: fused {tf:6.1f}   NCCL+GEMM {tn:6.1f}   (GEMM alone {tl:6.1f})")

    say(f"== distributed-optimizer step, DP{world}: fused kernels vs NCCL reduce-scatter + Adam + all-gather (ms per step)")
    from ..train.optimizer import DistributedOptimizer, OptimizerConfig
    from .state import ParallelDims, init_parallel_state

    ps = init_parallel_state(ParallelDims(dp=world))

    class _Flat(torch.nn.Module):
        def __init__(self, n):
            super().__init__()
            self.w = torch.nn.Parameter(torch.zeros(n, dtype=torch.bfloat16, device=dev))

    for n in (64 << 20, 512 << 20):
        res = {}
        for fused in (True, False):
            m = _Flat(n)
            opt = DistributedOptimizer(m, ps, OptimizerConfig(lr=1e-4, clip_grad=1.0, fused_dp=fused))
            m.w.main_grad.normal_(0, 1e-3)
            res[fused] = _time(lambda: opt.step(), 5, False, dev) / 1000
            del opt, m
            torch.cuda.empty_cache()
        say(f"  {n >> 20:5d} Mi parameters: fused {res[True]:7.2f}   NCCL {res[False]:7.2f}   "
            f"(link bytes per rank {(world - 1) * n // world * 6 / 1e9:.2f} GB)")

    say(f"== context-parallel attention, CP{world}: K/V (fwd) and Q/dO/dQ (bwd) cross NVLink once by peer stores")
    from .cp_peer import CPComm, peer_attention

    Hq, Hkv = 32, 8
    for L in (8192, 32768):
        cs = L // (2 * world)
        comm = CPComm(GroupInfo(dist.group.WORLD, tuple(range(world)), rank), dev, 2 * cs, Hq, Hkv)
        q = torch.randn(2 * cs, Hq, 128, device=dev).bfloat16().requires_grad_()
        k = torch.randn(2 * cs, Hkv, 128, device=dev).bfloat16().requires_grad_()
        v = torch.randn(2 * cs, Hkv, 128, device=dev).bfloat16().requires_grad_()
        do = torch.randn(2 * cs, Hq, 128, device=dev).bfloat16()
        tf = _time(lambda: peer_attention(q.detach(), k.detach(), v.detach(), comm, L), 5, False, dev)
        tfb = _time(lambda: peer_attention(q, k, v, comm, L).backward(do), 5, False, dev)
        # lower bound: this rank's share of the work if the whole sequence sat on one GPU
        qf = torch.randn(L, Hq, 128, device=dev).bfloat16().requires_grad_()
        kf = torch.randn(L, Hkv, 128, device=dev).bfloat16().requires_grad_()
        vf = torch.randn(L, Hkv, 128, device=dev).bfloat16().requires_grad_()
        dof = torch.randn(L, Hq, 128, device=dev).bfloat16()
        cu = torch.tensor([0, L], dtype=torch.int32, device=dev)
        t1 = _time(lambda: ops.attention_varlen(qf.detach(), kf.detach(), vf.detach(), cu), 5, False, dev)
        t1b = _time(lambda: ops.attention_varlen(qf, kf, vf, cu).backward(dof), 5, False, dev)
        say(f"  L={L:6d}: forward {tf:8.1f} us, forward+backward {tfb:8.1f} us   "
            f"(single-GPU attention of the whole sequence / {world}: {t1 / world:8.1f}, {t1b / world:8.1f})")
        comm.close()

    if args.timeline:
        for (M, K) in [(16, H // world), (128, F // world)]:
            x = torch.randn(M, K, device=dev).bfloat16()
            w = (torch.randn(H, K, device=dev) * 0.02).bfloat16()
            res = torch.randn(M, H, device=dev).bfloat16()
            nw = torch.ones(H, device=dev).bfloat16()
            for _ in range(3):
                comm.gemm_ar_add_rmsnorm(x, w, res, nw, 1e-6)
            torch.cuda.synchronize()
            dist.barrier()
            comm.timeline = torch.zeros(148, 8, dtype=torch.int64, device=dev)
            for _ in range(4):
                comm.gemm_ar_add_rmsnorm(x, w, res, nw, 1e-6)
            torch.cuda.synchronize()
            t = comm.timeline.cpu()
            comm.timeline = None
            t = t[t[:, 0] > 0]
            rel = (t[:, :6] - t[:, 0].min()).float() / 1000
            say(f"== phase stamps of the all-reduce kernel, M={M} K={K}, {t.shape[0]} CTAs (us: min / median / max)")
            for i, n in enumerate(["start", "tiles stored", "CTA barrier", "signalled", "peers arrived", "reduced"]):
                say(f"  {n:14s} {rel[:, i].min():7.2f} {rel[:, i].median():7.2f} {rel[:, i].max():7.2f}")
    C.check_error_flag(dev)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
