"""Headline benchmark: colocated GRPO step (rollout + train + weight sync) of a
Qwen3-8B-shaped model, tokens/s for the whole job.

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Config (weak scaling: per-GPU work fixed): per GPU 16 prompts of 512 random token
ids, 8 samples each, responses up to 2048 tokens at temperature 1; at 8 GPUs that
is the named configuration (128 prompts, trainer TP2 x DP4 with the distributed
optimizer, rollout TP2 x 4 engines).  Random-init weights, synthetic prompts,
parity reward, GRPO clip 0.2 with a k1 KL term (coef 0.001) to a frozen reference,
weight sync after every step.

`value` is device-timed (CUDA events around the K steps); `e2e.value` is wall
clock around the same public-API calls, which include, per step, the host->device
copy of that step's prompts from pinned memory and the device->host read of the
step's loss.

Wall-time budget: the whole run (start-up + warm-up + timed steps + teardown) is
planned to end inside `--time-budget-s` seconds (default 780, or the environment
variable RELAX_B200_BENCH_BUDGET_S).  After the first warm-up step its duration is
known; if W warm-up and K timed steps cannot fit, fewer are run - never less work
per step - and the line reports the counts really run next to `steps_requested`
and `warmup_requested`.  On SIGTERM rank 0 prints the line for the steps completed
so far (`"partial": true`) before leaving.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import threading
import time
import faulthandler

T_PROCESS_START = time.perf_counter()

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--prompts-per-gpu", type=int, default=16)
    ap.add_argument("--group-size", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--response-len", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=None, help="debug only: override depth (result is then not comparable)")
    ap.add_argument("--max-tokens-per-gpu", type=int, default=5120)
    ap.add_argument("--kv-gb", type=float, default=None)
    ap.add_argument("--tp", type=int, default=0, help="debug only: tensor-parallel size of trainer and engines (default 2 when N >= 2)")
    ap.add_argument("--cp", type=int, default=1,
                    help="context parallelism of the trainer (long-context config shape): world = tp x cp x dp; engines keep tp")
    ap.add_argument("--cp-attention", default=None, choices=["peer", "allgather"],
                    help="how context-parallel ranks see each other's K/V: NVLink staging buffers (default) or one all-gather")
    ap.add_argument("--ep", type=int, default=1,
                    help="expert parallelism of trainer and engines for MoE models (config 2 shape; sets tensor parallelism to 1)")
    ap.add_argument("--loss", default="grpo", choices=["grpo", "gspo"],
                    help="gspo: sequence-level ratio with clip 3e-4 / 4e-4 (the MoE config of the benchmark list)")
    ap.add_argument("--no-fused-tp", action="store_true",
                    help="A/B: use the NCCL statements instead of the fused GEMM+collective kernels (TP>1 only)")
    ap.add_argument("--time-budget-s", type=float, default=float(os.environ.get("RELAX_B200_BENCH_BUDGET_S", "780")),
                    help="wall-clock budget of the whole process; warm-up / timed step counts shrink to fit (0: no budget)")
    ap.add_argument("--decode-window", type=int, default=None, help="decode steps per host round trip in the rollout engine")
    ap.add_argument("--profile-host", action="store_true", help="debug: with --profile-kernels, also list the host-side operators by self CPU time")
    ap.add_argument("--profile-kernels", type=int, default=0,
                    help="debug: after the timed steps run ONE more step under torch.profiler and print rank 0's top N kernels "
                         "by device time to stderr (the extra step is not part of any reported number)")
    return ap.parse_args()


def reference_arm(args):
    """The reference needs Ray, Megatron-LM, TransformerEngine, SGLang and its data-plane
    package at run time; none of them is installed and none can be fetched offline."""
    why = "reference run-time dependencies (ray, megatron.core, transformer_engine, sglang, transfer_queue) are not installed and cannot be installed offline"
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import importlib

        missing = [m for m in ("ray", "megatron.core", "sglang", "transformer_engine") if importlib.util.find_spec(m.split(".")[0]) is None]
        if not missing:
            why = "reference dependencies import, but no offline recipe drives its Ray Serve deployment on this box"
        else:
            why = f"reference cannot run: missing {', '.join(missing)} (not installable offline)"
    except Exception as e:  # noqa: BLE001
        why = f"reference probe failed: {e!r}"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons of this process's GPU during the timed region."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag = index, [], False

    def run(self):
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.5)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    if os.environ.get("RELAX_B200_HANG_DUMP_S"):
        # debugging aid: print every thread's Python stack and exit if the run is still going after this many seconds
        faulthandler.dump_traceback_later(int(os.environ["RELAX_B200_HANG_DUMP_S"]), exit=True)
    import torch
    import torch.distributed as dist

    from relax_b200.algo.loss import LossConfig
    from relax_b200.models.config import get_config
    from relax_b200.ops import cuda as C
    from relax_b200.orchestration.colocate import ColocateConfig, ColocatedGRPO
    from relax_b200.train.actor import TrainConfig
    from relax_b200.train.optimizer import OptimizerConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    assert C.available()

    over = {} if args.layers is None else {"num_layers": args.layers}
    mcfg = get_config(args.model, **over)
    tp = args.tp if args.tp else (2 if world >= 2 else 1)
    ep = max(1, args.ep)
    if ep > 1:
        if not mcfg.is_moe or world % ep:
            raise SystemExit(f"--ep {ep} needs a MoE model and a world size it divides (world {world}, model {mcfg.name})")
        tp = 1
    gspo = args.loss == "gspo"
    cp = max(1, args.cp)
    if world % (tp * cp):
        raise SystemExit(f"--tp {tp} x --cp {cp} does not divide the world size {world}")
    G = args.group_size
    n_prompts = args.prompts_per_gpu * world
    kv_bytes_per_block = mcfg.num_layers * 2 * 16 * (mcfg.num_query_groups // tp) * mcfg.head_dim * 2
    ref_on_host = world == 1   # one GPU holds the whole model: park the frozen reference in pinned host memory
    kv_gb = args.kv_gb if args.kv_gb is not None else (52.0 if world == 1 else 40.0)
    kv_blocks = int(kv_gb * (1 << 30) / kv_bytes_per_block)
    need_blocks = args.prompts_per_gpu * tp * ep * G * ((args.prompt_len + args.response_len + 15) // 16 + 1)
    kv_blocks = min(kv_blocks, need_blocks)
    cfg = ColocateConfig(
        model=mcfg,
        train=TrainConfig(advantage_estimator="gspo" if gspo else "grpo", n_samples_per_prompt=G, global_batch_size=n_prompts * G,
                          max_tokens_per_gpu=args.max_tokens_per_gpu, pad_multiple=128, ref_on_host=ref_on_host,
                          cp_attention=args.cp_attention,
                          loss=LossConfig(eps_clip=3e-4 if gspo else 0.2, eps_clip_high=4e-4 if gspo else 0.2, use_kl_loss=True,
                                          kl_loss_coef=0.001, kl_loss_type="k1", advantage_estimator="gspo" if gspo else "grpo"),
                          optim=OptimizerConfig(lr=1e-6, clip_grad=1.0, grad_dtype="fp32")),
        trainer_tp=tp, rollout_tp=tp, trainer_cp=cp, trainer_ep=ep, rollout_ep=ep, rollout_batch_size=n_prompts, prompt_len=args.prompt_len,
        max_response_len=args.response_len, temperature=1.0, rm_type="parity", eos_token_id=None,
        kv_blocks=kv_blocks, kv_block_size=16, max_running=512, seed=0, rollout_seed=42,
        offload_rollout=True, release_rollout_weights=True, pinned_prompts=True,
        fused_tp=not args.no_fused_tp)
    if args.decode_window is not None:
        os.environ["RELAX_B200_DECODE_WINDOW"] = str(args.decode_window)
    run = ColocatedGRPO(cfg, device=dev)
    torch.cuda.synchronize()
    startup_s = time.perf_counter() - T_PROCESS_START
    budget = args.time_budget_s if args.time_budget_s > 0 else float("inf")
    TEARDOWN_RESERVE_S = 25.0

    def agree_max(x: float) -> float:
        """Every rank takes the same scheduling decision: the slowest rank's clock counts."""
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def elapsed() -> float:
        return time.perf_counter() - T_PROCESS_START

    # ---- warm-up: after the first step its cost is known and the rest of the run is planned against the budget
    warm_req, steps_req = args.warmup, args.steps
    warm_done, step_est = 0, 0.0
    plan_steps = steps_req
    while warm_done < warm_req:
        t_w = time.perf_counter()
        run.step()
        torch.cuda.synchronize()
        warm_done += 1
        step_est = agree_max(time.perf_counter() - t_w)
        left = budget - agree_max(elapsed()) - TEARDOWN_RESERVE_S
        fit = int(left // max(step_est, 1e-3))             # whole steps that still fit
        if fit >= (warm_req - warm_done) + steps_req:
            continue
        # not everything fits: keep at least one timed step, then up to three warm-up steps in total, then timed steps
        more_warm = max(0, min(warm_req, 3) - warm_done)
        more_warm = max(0, min(more_warm, fit - 1))
        plan_steps = max(1, min(steps_req, fit - more_warm))
        warm_req = warm_done + more_warm
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    sampler.start()
    C.reset_launch_count()
    mem0 = torch.cuda.memory_stats(dev)
    torch.cuda.reset_peak_memory_stats(dev)
    ev0 = torch.cuda.Event(enable_timing=True)
    step_events = []
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ev0.record()
    acc = {"resp": 0, "tot": 0, "sync_ms": [], "losses": [], "h2d": 0, "d2h": 0, "parts": {}, "lp_diff": None, "steps": 0,
           "wall": 0.0}

    def allocator_summary():
        """Caching-allocator traffic inside the timed region: device allocations (cudaMalloc calls) and retries
        (cache flushes under memory pressure) stall the host, so they explain device idle time."""
        m = torch.cuda.memory_stats(dev)
        return {"device_allocs": int(m.get("num_device_alloc", 0) - mem0.get("num_device_alloc", 0)),
                "device_frees": int(m.get("num_device_free", 0) - mem0.get("num_device_free", 0)),
                "alloc_retries": int(m.get("num_alloc_retries", 0) - mem0.get("num_alloc_retries", 0)),
                "peak_allocated_gb": round(m.get("allocated_bytes.all.peak", 0) / 2 ** 30, 1),
                "peak_reserved_gb": round(m.get("reserved_bytes.all.peak", 0) / 2 ** 30, 1)}

    def build_line(dev_s, wall, resp_all, tot_all, launches, n_steps, partial=False):
        value = resp_all / max(dev_s, 1e-9)
        out = {
            "metric": "grpo_e2e_response_tokens_per_sec_per_box",
            "value": round(value, 2), "unit": "tokens/s", "n_gpus": world, "steps": n_steps, "warmup": warm_done,
            "ms_per_step": round(dev_s * 1e3 / max(1, n_steps), 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic prompts (random token ids), random-init weights, parity reward",
            "config": {
                "model": mcfg.name + ("" if args.layers is None else f"-{args.layers}L-debug"),
                "global_batch": n_prompts, "group_size": G, "seq_len": args.prompt_len + args.response_len,
                "prompt_len": args.prompt_len, "max_response_len": args.response_len,
                "parallelism": (f"trainer tp{tp}xcp{cp}xdp{world // (tp * cp)} (distributed optimizer), rollout tp{tp}x{world // tp} engines, colocated"
                                if cp > 1 else
                                f"trainer tp{tp}xdp{world // tp} (distributed optimizer), rollout tp{tp}x{world // tp} engines, colocated"
                                if ep == 1 else
                                f"trainer ep{ep} x dp{world} (distributed optimizer), rollout ep{ep}x{world // ep} engines, colocated"),
                "loss": ("gspo sequence-level clip 3e-4/4e-4" if gspo else "grpo clip 0.2") + " + k1 kl 0.001 to frozen reference",
                "weight_sync_every_step": True,
                "cache": "working set per step (weights + activations + KV) far exceeds the 126 MB L2; no flush needed",
            },
            "steps_requested": steps_req, "warmup_requested": args.warmup, "time_budget_s": None if budget == float("inf") else budget,
            "startup_s": round(startup_s, 1),
            "total_tokens_per_sec": round(tot_all / max(dev_s, 1e-9), 2),
            "weight_sync_ms": round(sum(acc["sync_ms"]) / max(1, len(acc["sync_ms"])), 3),
            "phase_seconds_per_step": {k[5:]: round(v / max(1, n_steps), 3) for k, v in sorted(acc["parts"].items())},
            "loss": acc["losses"][-1] if acc["losses"] else None, "train_rollout_logprob_abs_diff": acc["lp_diff"],
            "e2e": {"value": round(resp_all / max(wall, 1e-9), 2), "unit": "tokens/s", "h2d_bytes_per_step": acc["h2d"] // max(1, n_steps),
                    "d2h_bytes_per_step": acc["d2h"] // max(1, n_steps)},
            "gpu_launches": launches,
            "allocator": allocator_summary(),
            "clocks": sampler.summary(),
        }
        if partial:
            out["partial"] = True
            out["note"] = "terminated by a signal: this rank's clock over the steps completed so far, not the max over ranks"
        return out

    printed = {"done": False}

    def on_term(signum, frame):
        # leave a line for what was measured; only completed steps count (their end events have been recorded)
        if rank == 0 and not printed["done"] and acc["steps"] > 0:
            printed["done"] = True
            try:
                ev = step_events[acc["steps"] - 1]
                dev_s = ev0.elapsed_time(ev) / 1e3 if ev.query() else acc["wall"]
            except Exception:  # noqa: BLE001
                dev_s = acc["wall"]
            print(json.dumps(build_line(dev_s, acc["wall"], acc["resp"] * world / tp / 1.0 if world > 1 else acc["resp"],
                                        acc["tot"] * world / tp if world > 1 else acc["tot"], C.launch_count(), acc["steps"], True)))
            sys.stdout.flush()
        os._exit(143)

    signal.signal(signal.SIGTERM, on_term)
    for i in range(plan_steps):
        if i > 0 and budget != float("inf"):
            # stop when one more step would pass the budget (the estimate follows the steps already timed)
            if agree_max(elapsed() + step_est) > budget - TEARDOWN_RESERVE_S:
                break
        t_s = time.perf_counter()
        m = run.step()
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        step_events.append(ev)
        acc["resp"] += m["response_tokens_local"]
        acc["tot"] += m["total_tokens_local"]
        acc["sync_ms"].append(m["weight_sync_ms"])
        acc["losses"].append(m["loss"])
        acc["lp_diff"] = next((float(v) for k, v in m.items() if k.endswith("train_rollout_logprob_abs_diff")), None)
        acc["h2d"] += m.get("h2d_bytes", 0)
        acc["d2h"] += m.get("d2h_bytes", 0)
        for k, v in m.items():
            if k.startswith("perf/"):
                acc["parts"][k] = acc["parts"].get(k, 0.0) + v
        acc["steps"] += 1
        acc["wall"] = time.perf_counter() - t0
        step_est = max(step_est * 0.5, time.perf_counter() - t_s)
    n_steps = acc["steps"]
    ev1 = step_events[-1]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - t0
    dev_s = ev0.elapsed_time(ev1) / 1e3
    sampler.stop_flag = True
    launches = C.launch_count()
    # each engine's TP ranks hold identical samples: count every sequence once
    stat = torch.tensor([dev_s, wall, acc["resp"] / tp, acc["tot"] / tp, float(launches)], device=dev, dtype=torch.float64)
    if world > 1:
        mx = stat.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stat.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        dev_s, wall = float(mx[0]), float(mx[1])
        resp_all, tot_all = float(sm[2]), float(sm[3])
        launches = int(mx[4])
    else:
        resp_all, tot_all = acc["resp"], acc["tot"]
    C.check_error_flag()
    signal.signal(signal.SIGTERM, signal.SIG_DFL)
    if rank == 0 and not printed["done"]:
        printed["done"] = True
        print(json.dumps(build_line(dev_s, wall, resp_all, tot_all, launches, n_steps)))
    sys.stdout.flush()
    if args.profile_kernels > 0:
        from torch.profiler import ProfilerActivity, profile

        acts = [ProfilerActivity.CUDA] + ([ProfilerActivity.CPU] if args.profile_host else [])
        with profile(activities=acts) as prof:
            t_p = time.perf_counter()
            run.step()
            torch.cuda.synchronize()
            t_p = time.perf_counter() - t_p
        if rank == 0:
            rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)
            tot = sum(e.device_time_total for e in rows)
            print(f"[profile] one extra step under the profiler: {t_p:.3f} s wall, {tot / 1e6:.3f} s of kernel time on rank 0", file=sys.stderr)
            for e in rows[:args.profile_kernels]:
                print(f"[profile] {e.device_time_total / 1e3:10.2f} ms {100 * e.device_time_total / max(tot, 1):5.1f}% x{e.count:6d}  {e.key[:110]}",
                      file=sys.stderr)
            if args.profile_host:
                host = sorted(prof.key_averages(), key=lambda e: -e.self_cpu_time_total)
                tot_h = sum(e.self_cpu_time_total for e in host)
                print(f"[profile] host: {tot_h / 1e6:.3f} s of self CPU time in profiled operators", file=sys.stderr)
                for e in host[:args.profile_kernels]:
                    print(f"[profile]   host {e.self_cpu_time_total / 1e3:9.2f} ms x{e.count:6d} (mean {e.self_cpu_time_total / max(e.count, 1):7.1f} us)  {e.key[:90]}",
                          file=sys.stderr)
            # where the device sat idle: for every kernel, the time since the latest end of any earlier kernel
            from torch.autograd import DeviceType

            ks = sorted((e for e in prof.events() if e.device_type == DeviceType.CUDA and e.time_range is not None),
                        key=lambda e: e.time_range.start)
            idle, last_end, last_name = {}, None, ""
            for e in ks:
                st, en = e.time_range.start, e.time_range.end
                if last_end is not None and st > last_end:
                    g = idle.setdefault(last_name[:48] + "  ->  " + e.name[:48], [0.0, 0])
                    g[0] += st - last_end
                    g[1] += 1
                if last_end is None or en >= last_end:
                    last_end, last_name = en, e.name
            tot_idle = sum(v[0] for v in idle.values())
            print(f"[profile] device idle between kernels: {tot_idle / 1e6:.3f} s; by (last kernel before the gap -> first after):", file=sys.stderr)
            for name, (us, n) in sorted(idle.items(), key=lambda kv: -kv[1][0])[:16]:
                print(f"[profile]   idle {us / 1e3:9.2f} ms x{n:6d} (mean {us / max(n, 1):7.1f} us)  {name}", file=sys.stderr)
    run.close()
    if world > 1:
        from relax_b200.parallel.state import shutdown_distributed

        shutdown_distributed(timeout_s=120.0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
