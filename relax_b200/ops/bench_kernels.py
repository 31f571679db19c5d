"""Kernel-level benchmark of the sm_100a operators, with roofline fractions.

    python -m relax_b200.ops.bench_kernels                       # every section, training + decode shapes of Qwen3-8B
    python -m relax_b200.ops.bench_kernels --only gemm --tokens 2048 --iters 3 --warmup 1   # a small case for a profiler

Times come from CUDA events on the launching stream after warm-up; inputs are rotated through a
pool larger than the L2 cache where a kernel's working set would otherwise fit in it.  Fractions
are reported against a measured copy bandwidth and a measured cuBLAS bf16 GEMM rate given with
``--peaks FILE`` (JSON with ``hbm_gbs`` and ``bf16_tflops``); without the file the absolute
numbers are printed alone.  Library kernels (cuBLAS through ``torch.matmul``, flash-attn 2 when
importable) are timed beside ours as the comparison arm.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _timeit(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters   # ms


class _Peaks:
    def __init__(self, path):
        self.hbm = self.tf = None
        if path and os.path.exists(path):
            d = json.load(open(path))
            self.hbm, self.tf = d.get("hbm_gbs"), d.get("bf16_tflops")

    def flops(self, tflops):
        return f"{tflops:7.1f} TFLOP/s" + (f" ({tflops / self.tf:.2f} of measured cuBLAS peak)" if self.tf else "")

    def bytes(self, gbs):
        return f"{gbs:7.1f} GB/s" + (f" ({gbs / self.hbm:.2f} of measured copy bandwidth)" if self.hbm else "")


def bench_gemm(args, pk):
    from . import cuda as C

    T, dev = args.tokens, "cuda"
    print(f"== GEMM, {T} tokens (ms | TFLOP/s): ours vs cuBLAS")
    shapes = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (24576, 4096), "down": (4096, 12288)}
    for name, (N, K) in shapes.items():
        a = torch.randn(T, K, device=dev).bfloat16()
        w = torch.randn(N, K, device=dev).bfloat16()
        dy = torch.randn(T, N, device=dev).bfloat16()
        mg = torch.zeros(N, K, device=dev)
        fl = 2 * T * N * K / 1e9
        rows = [("fwd  x W^T", lambda: C.matmul_nt(a, w), lambda: a @ w.t()),
                ("dgrad dy W", lambda: C.matmul_nn(dy, w), lambda: dy @ w),
                ("wgrad dy^T x -> fp32 +=", lambda: C.matmul_tn(dy, a, out=mg, accumulate=True), lambda: dy.t() @ a)]
        for label, ours, lib in rows:
            t, tl = _timeit(ours, args.iters, args.warmup), _timeit(lib, args.iters, args.warmup)
            print(f"  {name:8s} {label:24s} {t:7.3f} ms {pk.flops(fl / t)} | cuBLAS {tl:7.3f} ms {fl / tl:7.1f}")


def bench_gemm_fp8(args, pk):
    from .. import ops
    from . import cuda as C

    T, dev = args.tokens, "cuda"
    print(f"== block-scaled fp8 GEMM (e4m3, 1x128 / 128x128 scales), {T} tokens: ours fp8 vs ours bf16")
    for name, (N, K) in {"qkv": (6144, 4096), "gate_up": (24576, 4096), "down": (4096, 12288)}.items():
        a = torch.randn(T, K, device=dev).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
        wq, ws = ops.blockwise_cast_to_fp8(w, 128)
        aq, as_ = C.quantize_rows_fp8(a)
        fl = 2 * T * N * K / 1e9
        t8 = _timeit(lambda: C.fp8_linear(a, wq, ws, aq, as_), args.iters, args.warmup)
        t16 = _timeit(lambda: C.matmul_nt(a, w), args.iters, args.warmup)
        print(f"  {name:8s} fp8 {t8:7.3f} ms {fl / t8:7.1f} TFLOP/s | bf16 {t16:7.3f} ms {fl / t16:7.1f} TFLOP/s")


def bench_attention(args, pk):
    from .. import ops

    T, dev, nq, nkv, hd = args.tokens, "cuda", 32, 8, 128
    seq = args.seq_len
    n = max(1, T // seq)
    cu = torch.arange(0, (n + 1) * seq, seq, device=dev, dtype=torch.int32)
    T = n * seq
    q = torch.randn(T, nq, hd, device=dev).bfloat16().requires_grad_()
    k = torch.randn(T, nkv, hd, device=dev).bfloat16().requires_grad_()
    v = torch.randn(T, nkv, hd, device=dev).bfloat16().requires_grad_()
    fl_f = n * 4 * seq * seq / 2 * nq * hd / 1e9   # causal forward
    tf = _timeit(lambda: ops.attention_varlen(q.detach(), k.detach(), v.detach(), cu), args.iters, args.warmup)
    do = torch.randn(T, nq, hd, device=dev).bfloat16()

    def fb():
        ops.attention_varlen(q, k, v, cu).backward(do)

    tfb = _timeit(fb, args.iters, args.warmup)
    print(f"== causal flash attention, {n} x {seq} tokens, {nq}/{nkv} heads x {hd}")
    print(f"  forward            {tf:7.3f} ms {pk.flops(fl_f / tf)}")
    print(f"  forward + backward {tfb:7.3f} ms   backward alone {pk.flops(2.5 * fl_f / max(tfb - tf, 1e-6))}")
    try:
        from flash_attn import flash_attn_varlen_func as fa2

        t2 = _timeit(lambda: fa2(q.detach(), k.detach(), v.detach(), cu, cu, seq, seq, causal=True), args.iters, args.warmup)

        def fb2():
            fa2(q, k, v, cu, cu, seq, seq, causal=True).backward(do)

        print(f"  flash-attn 2 (library): forward {t2:7.3f} ms, forward + backward {_timeit(fb2, args.iters, args.warmup):7.3f} ms")
    except Exception as e:  # noqa: BLE001
        print(f"  flash-attn 2 not importable here ({type(e).__name__})")


def bench_decode(args, pk):
    from . import cuda as C

    B, dev, nq, nkv, hd, bs = args.batch, "cuda", 32, 8, 128, 16
    print(f"== decode, batch {B}")
    for ctxlen in (600, 1500, 2500):
        nb = (2560 + bs - 1) // bs
        kc = torch.randn(B * nb + 1, bs, nkv, hd, device=dev).bfloat16()
        vc = torch.randn_like(kc)
        bt = torch.arange(B * nb, device=dev, dtype=torch.int32).view(B, nb)
        ctx = torch.full((B,), ctxlen, device=dev, dtype=torch.int32)
        q = torch.randn(B, nq, hd, device=dev).bfloat16()
        byts = 2 * B * ctxlen * nkv * hd * 2
        for ver in (3, 1):
            t = _timeit(lambda: C.paged_decode_attention(q, kc, vc, bt, ctx, max_ctx=2560, version=ver), args.iters, args.warmup)
            name = "tcgen05" if ver == 3 else "CUDA-core"
            print(f"  paged attention ctx {ctxlen:5d} ({name:9s}) {t * 1e3:7.1f} us {pk.bytes(byts / t / 1e6)}")
    for name, (N, K) in {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (24576, 4096), "down": (4096, 12288)}.items():
        x = torch.randn(B, K, device=dev).bfloat16()
        ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(6)]   # > L2 in total
        i = [0]

        def ours():
            i[0] = (i[0] + 1) % len(ws)
            with torch.no_grad():
                return C.linear(x, ws[i[0]])

        def lib():
            i[0] = (i[0] + 1) % len(ws)
            return torch.matmul(x, ws[i[0]].t())

        t, tl = _timeit(ours, args.iters, args.warmup), _timeit(lib, args.iters, args.warmup)
        print(f"  skinny GEMM {name:8s} {t * 1e3:7.1f} us {pk.bytes(N * K * 2 / t / 1e6)} | cuBLAS {tl * 1e3:7.1f} us")
    V = 151936
    logits = torch.randn(B, V, device=dev).bfloat16()     # what the rollout LM head writes
    from .. import ops

    temp = torch.ones(B, device=dev)
    tk = torch.full((B,), -1, device=dev, dtype=torch.int64)
    tp = torch.ones(B, device=dev)
    u = torch.rand(B, device=dev)
    t = _timeit(lambda: ops.sample(logits, temp, tk, tp, u), args.iters, args.warmup)
    print(f"  sampling (temperature/top-k/top-p, V={V}, bf16 logits) {t * 1e3:7.1f} us {pk.bytes(B * V * 2 / t / 1e6)}")


def bench_lm_head(args, pk):
    from . import cuda as C

    T, H, V, dev = min(args.tokens, 4096), 4096, 151936, "cuda"
    h = torch.randn(T, H, device=dev).bfloat16().requires_grad_()
    w = (torch.randn(V, H, device=dev) * 0.02).bfloat16().requires_grad_()
    tgt = torch.randint(0, V, (T,), device=dev)
    fl = 2 * T * V * H / 1e9
    tf = _timeit(lambda: C.fused_lm_head_logprob(h.detach(), w.detach(), tgt), args.iters, args.warmup)

    def fb():
        lp, ent = C.fused_lm_head_logprob(h, w, tgt)
        (lp.sum() + 0.01 * ent.sum()).backward()

    tfb = _timeit(fb, max(1, args.iters // 2), args.warmup)
    print(f"== fused LM head (log-prob + entropy, logits never stored), {T} rows x V={V}")
    print(f"  forward            {tf:7.3f} ms {pk.flops(fl / tf)}")
    print(f"  forward + backward {tfb:7.3f} ms {pk.flops(4 * fl / tfb)} (forward + recompute + dgrad + wgrad)")


def bench_elementwise(args, pk):
    from .. import ops
    from . import reference as R

    T, H, F, dev, nq, hd = args.tokens, 4096, 12288, "cuda", 32, 128
    x = torch.randn(T, H, device=dev).bfloat16()
    w = torch.ones(H, device=dev).bfloat16()
    gu = torch.randn(T, 2 * F, device=dev).bfloat16()
    pos = torch.arange(T, device=dev)
    cos, sin = R.rope_cos_sin(pos, hd, 1e6)
    qq = torch.randn(T, nq, hd, device=dev).bfloat16()
    print(f"== memory-bound kernels, {T} tokens")
    rows = [("rmsnorm", lambda: ops.rmsnorm(x, w), 2 * T * H * 2),
            ("add + rmsnorm", lambda: ops.add_rmsnorm(x, x, w), 4 * T * H * 2),
            ("swiglu", lambda: ops.swiglu(gu), 3 * T * F * 2),
            ("rope (q heads)", lambda: ops.apply_rope(qq, cos, sin), 2 * T * nq * hd * 2)]
    for name, fn, byts in rows:
        t = _timeit(fn, args.iters, args.warmup)
        print(f"  {name:16s} {t * 1e3:7.1f} us {pk.bytes(byts / t / 1e6)}")


def bench_train_step(args, pk):
    """Kernel-time breakdown of one training micro-batch (forward + backward) of a few Qwen3-8B layers."""
    from torch.profiler import ProfilerActivity, profile

    from ..algo.loss import LossConfig
    from ..models.config import get_config
    from ..train.actor import TrainActor, TrainConfig
    from ..train.optimizer import OptimizerConfig

    cfg = get_config("qwen3-8b", num_layers=args.layers)
    actor = TrainActor(cfg, TrainConfig(max_tokens_per_gpu=args.tokens, pad_multiple=128, loss=LossConfig(eps_clip=0.2),
                                        optim=OptimizerConfig(lr=1e-6, grad_dtype="fp32")), device="cuda", seed=0)
    n = max(1, args.tokens // args.seq_len)
    toks = [torch.randint(0, 150000, (args.seq_len,)).tolist() for _ in range(n)]
    pb = actor._pack(toks, [args.seq_len - 512] * n)

    def step():
        lp, en = actor._forward_logp(pb, True)
        (lp.sum() + 0.01 * en.sum()).backward()

    t = _timeit(step, args.iters, args.warmup)
    print(f"== training micro-batch, {n} x {args.seq_len} tokens, {args.layers} layers + LM head: {t:.2f} ms forward + backward")
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize()
    ev = prof.key_averages()
    tot = sum(r.device_time_total for r in ev)
    for r in sorted(ev, key=lambda r: -r.device_time_total)[:16]:
        print(f"  {r.device_time_total / 1000:8.3f} ms {100 * r.device_time_total / tot:5.1f}%  x{r.count:4d}  {r.key[:96]}")


def bench_moe(args, pk):
    """Grouped expert GEMMs of a Qwen3-30B-A3B layer on one EP rank (16 local experts, hidden 2048, expert FFN 768):
    one launch for all experts against a loop of library GEMMs over the same expert-sorted rows."""
    from .. import ops
    from ..models.moe import padded_expert_layout

    dev, E, H, F = "cuda", 16, 2048, 768
    rows = args.tokens * 8 // 8                      # tokens x top-8 spread over 8 EP ranks
    g = torch.Generator(device=dev).manual_seed(0)
    e_of = torch.randint(0, E, (rows,), device=dev, generator=g)
    x = torch.randn(rows, H, device=dev, generator=g).bfloat16()
    w1 = (torch.randn(E, 2 * F, H, device=dev, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn(E, H, F, device=dev, generator=g) * 0.02).bfloat16()
    order, dest, cap, tile_expert, expert_rows = padded_expert_layout(e_of, E)
    xp = x.new_zeros(cap, H).index_copy(0, dest, x[order])
    counts = torch.bincount(e_of, minlength=E).tolist()
    xs = x[order]

    def ours():
        with torch.no_grad():
            a = ops.swiglu(ops.grouped_linear(xp, w1, tile_expert, expert_rows))
            return ops.grouped_linear(a, w2, tile_expert, expert_rows)

    def lib():
        o, outs = 0, []
        for e, n in enumerate(counts):
            h = torch.matmul(xs[o:o + n], w1[e].t())
            a = torch.nn.functional.silu(h[:, :F]) * h[:, F:]
            outs.append(torch.matmul(a, w2[e].t()))
            o += n
        return outs

    t, tl = _timeit(ours, args.iters, args.warmup), _timeit(lib, args.iters, args.warmup)
    fl = 2 * rows * (2 * F * H + H * F) / 1e9
    print(f"== MoE expert MLPs, {rows} routed rows over {E} local experts (H {H}, F {F})")
    print(f"  grouped GEMMs + SwiGLU (3 launches)   {t:7.3f} ms {pk.flops(fl / t)} | loop of library GEMMs ({3 * E} launches) {tl:7.3f} ms")


def bench_decode_step(args, pk):
    """One whole decode step of the rollout engine (all layers + LM head + sampling + device-side advance) as the
    engine runs it: a CUDA graph replayed back to back.  Reports ms per step against the bytes a step must read
    (weights + KV cache of the batch) and the per-kernel shares of one replay."""
    from torch.profiler import ProfilerActivity, profile

    from ..models.config import get_config
    from ..rollout.engine import RolloutEngine, SamplingParams

    cfg = get_config("qwen3-8b", num_layers=args.decode_layers)
    B, ctx, bs = args.batch, args.ctx, 16
    blocks = B * ((ctx + 64 + bs - 1) // bs + 1) + 8
    eng = RolloutEngine(cfg, device="cuda", dtype=torch.bfloat16, num_kv_blocks=blocks, block_size=bs, max_running=B,
                        max_model_len=ctx + 64, decode_window=args.window, memory_saver=False)
    eng.weights.flat.normal_(0, 0.02)
    for k, v in eng.weights.p.items():
        if "norm" in k:
            v.fill_(1.0)
    eng.kv.normal_(0, 1.0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (ctx,), generator=g).tolist() for _ in range(B)]
    sp = SamplingParams(max_new_tokens=64, ignore_eos=True)
    for p_ in prompts:
        eng.add_request(p_, sp)
    while eng.waiting:          # prefill everything
        eng.step()
    eng.step()                  # first window: captures the graph
    torch.cuda.synchronize()
    st = eng._graphs[next(b for b in eng.GRAPH_BUCKETS if b >= B)]
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = args.window
    s.record()
    for _ in range(n):
        st["graph"].replay()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / n
    wbytes = sum(v.numel() * 2 for k, v in eng.weights.p.items() if k != "embed")
    kvbytes = 2 * B * (ctx + 4) * (cfg.num_query_groups * cfg.head_dim) * 2 * cfg.num_layers
    print(f"== decode step, batch {B}, context {ctx}, {cfg.num_layers} layers: {ms:.3f} ms per step (graph replay), "
          f"{pk.bytes((wbytes + kvbytes) / ms / 1e6)} over weights {wbytes / 1e9:.2f} GB + KV {kvbytes / 1e9:.2f} GB")
    import time as _t

    t0 = _t.perf_counter()
    for _ in range(3):
        eng.step()
    torch.cuda.synchronize()
    print(f"   engine.step() with a window of {args.window}: {(_t.perf_counter() - t0) / (3 * args.window) * 1e3:.3f} ms per decode step, host included")
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        st["graph"].replay()
        torch.cuda.synchronize()
    ev = prof.key_averages()
    tot = sum(r.device_time_total for r in ev)
    for r in sorted(ev, key=lambda r: -r.device_time_total)[:14]:
        print(f"  {r.device_time_total / 1000:8.3f} ms {100 * r.device_time_total / tot:5.1f}%  x{r.count:4d}  {r.key[:110]}")


SECTIONS = {"decode_step": bench_decode_step, "moe": bench_moe, "gemm": bench_gemm, "gemm_fp8": bench_gemm_fp8, "attention": bench_attention, "decode": bench_decode, "lm_head": bench_lm_head,
            "elementwise": bench_elementwise, "train_step": bench_train_step}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--only", choices=sorted(SECTIONS), default=None)
    ap.add_argument("--tokens", type=int, default=5120, help="rows of the training-shape problems")
    ap.add_argument("--seq-len", type=int, default=2560)
    ap.add_argument("--batch", type=int, default=80, help="decode batch")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=4, help="transformer layers of the train_step section")
    ap.add_argument("--decode-layers", type=int, default=36, help="layers of the decode_step section")
    ap.add_argument("--ctx", type=int, default=1536, help="context length of the decode_step section")
    ap.add_argument("--window", type=int, default=16, help="decode steps per host round trip (decode_step section)")
    ap.add_argument("--peaks", default="MEASURED_PEAKS.json")
    args = ap.parse_args()
    pk = _Peaks(args.peaks)
    torch.manual_seed(0)
    for name, fn in SECTIONS.items():
        if args.only == name or (args.only is None and name not in ("train_step", "decode_step")):
            fn(args, pk)


if __name__ == "__main__":
    main()
