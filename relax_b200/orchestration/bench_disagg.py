"""Fully-asynchronous RL on disjoint GPU pools, timed: tokens/s, trainer idle fraction and weight-sync cost for the
NVLink peer-store push and for the NCCL-broadcast arm.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29520 \
        -m relax_b200.orchestration.bench_disagg --train-gpus 2 --trainer-tp 2 --rollout-tp 1 --layers 8

The first ``--train-gpus`` ranks train, the rest are rollout engines of ``--rollout-tp`` ranks each; a rollout may
run ``--max-staleness`` steps ahead of the trainer.  Each arm (``peer``, ``broadcast``) runs ``--num-rollout`` steps of
a Qwen3-8B-shaped model (``--layers`` deep) with synthetic prompts; rank 0 prints one JSON line per arm.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--train-gpus", type=int, default=2)
    ap.add_argument("--trainer-tp", type=int, default=2)
    ap.add_argument("--rollout-tp", type=int, default=1)
    ap.add_argument("--prompts", type=int, default=16, help="prompts per rollout step, all engines together")
    ap.add_argument("--group-size", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--response-len", type=int, default=256)
    ap.add_argument("--num-rollout", type=int, default=4)
    ap.add_argument("--max-staleness", type=int, default=1)
    ap.add_argument("--arms", default="peer,broadcast")
    ap.add_argument("--image-side", type=int, default=0,
                    help="vision-language models: patches per side of the synthetic image in every prompt (32 = 448 x 448 pixels = 256 tokens)")
    a = ap.parse_args(argv)

    from ..algo.loss import LossConfig
    from ..models.config import get_config
    from ..parallel.state import shutdown_distributed
    from ..train.actor import TrainConfig
    from ..train.optimizer import OptimizerConfig
    from .disagg import DisaggConfig, DisaggregatedRL

    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist.init_process_group("gloo")
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = f"cuda:{local}" if cuda else "cpu"
    mcfg = get_config(a.model, num_layers=a.layers)
    tr, ro = tuple(range(a.train_gpus)), tuple(range(a.train_gpus, world))
    n_eng = len(ro) // a.rollout_tp
    seqs = a.prompts * a.group_size // n_eng
    blocks = seqs * ((a.prompt_len + a.response_len) // 16 + 2) + 16
    for i, arm in enumerate(a.arms.split(",")):
        cfg = DisaggConfig(
            model=mcfg, image_grid_side=a.image_side,
            train=TrainConfig(n_samples_per_prompt=a.group_size, global_batch_size=a.prompts * a.group_size,
                                          max_tokens_per_gpu=8192, pad_multiple=128 if cuda else 1,
                                          freeze_params_name_list=[r"^vision\."] if mcfg.vision is not None else None,
                                          loss=LossConfig(eps_clip=0.2, use_kl_loss=True, kl_loss_coef=0.001),
                                          optim=OptimizerConfig(lr=1e-6)),
            trainer_ranks=tr, rollout_ranks=ro, trainer_tp=a.trainer_tp, rollout_tp=a.rollout_tp,
            rollout_batch_size=a.prompts, prompt_len=a.prompt_len, max_response_len=a.response_len, kv_blocks=blocks,
            num_rollout=a.num_rollout, max_staleness=a.max_staleness, weight_push=arm, tag=f"b{os.environ.get('MASTER_PORT', '0')}{i}")
        rl = DisaggregatedRL(cfg, device=dev)
        rl.run()
        if cuda:
            torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            st = rl.stats
            sync = st["sync_ms"][1:] or st["sync_ms"]          # the first push also maps the peers' buffers
            kern = st["push_kernel_ms"][1:] or st["push_kernel_ms"]
            print(json.dumps({
                "arm": arm, "model": f"{mcfg.name}-{a.layers}L", "trainer": f"tp{a.trainer_tp}xdp{a.train_gpus // a.trainer_tp}",
                "rollout": f"{n_eng} engines x tp{a.rollout_tp}", "max_staleness": a.max_staleness, "steps": a.num_rollout,
                "response_tokens_per_s": round(st["tokens_per_s"], 1), "trainer_idle_fraction": round(st["trainer_idle_fraction"], 3),
                "weight_sync_ms_mean": round(sum(sync) / len(sync), 3), "push_kernel_ms_mean": round(sum(kern) / len(kern), 3),
                "bytes_per_push_per_trainer_rank": getattr(rl.pusher, "bytes_per_push", None)}), flush=True)
        rl.close()
    shutdown_distributed()
    return 0


if __name__ == "__main__":
    sys.exit(main())
