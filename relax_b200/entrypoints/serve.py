"""Stand-alone control-plane services: ``python -m relax_b200.entrypoints.serve <service> [--host H] [--port P]``.

* ``metrics``     - the metrics service (``/log_metric``, ``/log_metrics_batch``, ``/report_step``, ``/log_error``) with the
  tracking adapters chosen by the usual flags (relax/entrypoints/deploy_metrics_service.py);
* ``coordinator`` - the weight-sync coordinator (register / heartbeat / topology / weight-metadata long poll,
  relax/checkpoint_service/coordinator/service.py);
* ``viewer``      - the rollout result viewer (relax/entrypoints/visualize.py);
* ``engine``      - one rollout engine behind HTTP (``/generate``, ``/flush_cache``, ``/pause_generation``,
  ``/continue_generation``, ``/abort_request``, ``/get_server_info``; relax/backends/sglang/sglang_engine.py talks to
  its engines over the same surface); weights from ``--hf-checkpoint``;
* ``router``      - the request router as an HTTP proxy in front of engine servers (least loaded / sticky by key,
  health probes, ``/add_worker`` ``/remove_worker`` ``/list_workers``; relax/engine/router/router.py);
* ``teacher``     - an on-policy-distillation teacher: ``POST /score`` returns the teacher's log-probs of the response
  tokens (``--model-name`` / ``--hf-checkpoint`` choose it; ``--opd-teacher-urls`` of the training job point here).

Each serves until interrupted; the bound address is printed first so that launch scripts can read it.
"""
from __future__ import annotations

import argparse
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="relax_b200 control-plane services")
    ap.add_argument("service", choices=["metrics", "coordinator", "viewer", "teacher", "router", "engine"])
    ap.add_argument("--kv-blocks", type=int, default=4096, help="engine: KV-cache blocks of 16 tokens")
    ap.add_argument("--speculative-steps", type=int, default=0,
                    help="engine: proposals per pass drafted by the model's multi-token-prediction block (0 = off)")
    ap.add_argument("--workers", nargs="*", default=None, help="router: base URLs of the engine servers to start with")
    ap.add_argument("--router-timeout", type=float, default=600.0)
    ap.add_argument("--router-health-check-failure-threshold", type=int, default=3)
    ap.add_argument("--model-name", default="tiny", help="teacher: model preset")
    ap.add_argument("--hf-checkpoint", default=None, help="teacher: Hugging Face directory with the teacher's weights")
    ap.add_argument("--device", default=None, help="teacher: cuda / cpu (default: cuda when available)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--dir", default=None, help="viewer: dump directory; metrics: output directory of metrics.jsonl")
    ap.add_argument("--use-tensorboard", action="store_true")
    ap.add_argument("--max-seconds", type=float, default=None, help="leave after this long (tests, batch jobs)")
    a = ap.parse_args(argv)
    if a.service == "metrics":
        from ..metrics.adapters import build_adapters
        from ..metrics.service import MetricsService, serve

        ns = argparse.Namespace(metrics_dir=a.dir, save=None, use_tensorboard=a.use_tensorboard, log_to_console=True)
        srv, _ = serve(MetricsService(build_adapters(ns)), a.host, a.port)
    elif a.service == "coordinator":
        from ..weight_sync.dcs import Coordinator, serve

        srv, _ = serve(Coordinator(), a.host, a.port)
    elif a.service == "router":
        from ..rollout.router import Router, serve_router

        r = Router(max_failures=a.router_health_check_failure_threshold)
        for u in a.workers or []:
            r.add_worker(u)
        srv, _, _ = serve_router(r, a.host, a.port, timeout_s=a.router_timeout)
    elif a.service == "engine":
        import torch

        from ..models.config import get_config
        from ..rollout.engine import RolloutEngine
        from ..rollout.http_server import EngineServer

        dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
        cfg = get_config(a.model_name)
        eng = RolloutEngine(cfg, device=dev, dtype=torch.bfloat16 if dev.startswith("cuda") else torch.float32,
                            num_kv_blocks=a.kv_blocks, block_size=16, seed=a.seed, speculative=a.speculative_steps > 0,
                            speculative_steps=max(1, a.speculative_steps))
        if a.hf_checkpoint:
            from ..checkpoint import hf as H

            H.validate_against_hf(cfg, a.hf_checkpoint)
            H.load_hf_into_rollout(a.hf_checkpoint, cfg, eng.weights)
        es = EngineServer(eng, a.host, a.port)
        srv = es.httpd
    elif a.service == "teacher":
        import torch

        from ..algo.opd import InProcessTeacher, serve_teacher
        from ..models.config import get_config
        from ..train.actor import TrainActor, TrainConfig

        dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
        cfg = get_config(a.model_name)
        actor = TrainActor(cfg, TrainConfig(), device=dev, seed=a.seed, with_optimizer=False)
        if a.hf_checkpoint:
            from ..checkpoint import hf as H

            H.validate_against_hf(cfg, a.hf_checkpoint)
            H.load_hf_into_model(a.hf_checkpoint, cfg, actor.ps, actor.model)
        srv, _ = serve_teacher(InProcessTeacher(actor), a.host, a.port)
    else:
        from ..utils.visualize import serve_in_thread

        if not a.dir:
            ap.error("viewer needs --dir")
        srv, _ = serve_in_thread(a.dir, a.host, a.port)
    print(f"{a.service} listening on http://{srv.server_address[0]}:{srv.server_address[1]}", flush=True)
    t0 = time.monotonic()
    try:
        while a.max_seconds is None or time.monotonic() - t0 < a.max_seconds:
            time.sleep(0.2)
    except KeyboardInterrupt:
        pass
    srv.shutdown()
    srv.server_close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
