"""``python -m relax_b200.entrypoints.train <flags>`` (one process per GPU under ``torch.distributed.run``).

Parses the flag table, joins the process group, starts the metrics service with the requested
tracking adapters, builds the controller for the chosen mode and runs the training loop; the
counterpart of relax/entrypoints/train.py:81-126 without the Ray bring-up.
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    from ..config.arguments import parse_args
    from ..metrics.adapters import build_adapters
    from ..metrics.service import MetricsService
    from ..orchestration.controller import Controller

    args = parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    use_cuda = torch.cuda.is_available()
    if world > 1 and not dist.is_initialized():
        import datetime

        minutes = getattr(args, "distributed_timeout_minutes", None)
        kw = {"timeout": datetime.timedelta(minutes=minutes)} if minutes else {}
        if use_cuda:
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            dist.init_process_group(args.distributed_backend or "nccl", device_id=torch.device("cuda", local), **kw)
        else:
            dist.init_process_group("gloo", **kw)
    rank = dist.get_rank() if dist.is_initialized() else 0
    metrics = MetricsService(build_adapters(args) if rank == 0 else [])
    ctl = Controller(args, metrics)
    try:
        ctl.training_loop()
    finally:
        ctl.shutdown()
        if dist.is_initialized():
            from ..parallel.state import shutdown_distributed

            shutdown_distributed(timeout_s=30.0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
