"""Metrics service, adapters, FLOPs counter, profiler wrapper (CPU)."""
import json
import os

import torch

from relax_b200.metrics.adapters import JsonlAdapter
from relax_b200.metrics.flops import forward_flops, mfu, train_step_flops
from relax_b200.metrics.service import MetricsClient, MetricsService, serve
from relax_b200.models.config import get_config
from relax_b200.utils.profiler import TrainProfiler


def test_service_merges_roles_and_flushes_in_order(tmp_path):
    path = tmp_path / "m.jsonl"
    svc = MetricsService([JsonlAdapter(str(path))])
    svc.log_metric(1, "rollout/tokens", 10, "sum")
    svc.log_metric(1, "rollout/tokens", 5, "sum")
    svc.log_metric(0, "train/loss", 2.0)
    svc.log_metric(1, "train/loss", 1.0, "mean")
    svc.log_metric(1, "train/loss", 3.0, "mean")
    svc.log_metrics_batch(2, {"a": 1.0})
    svc.report_step(1)
    hist = svc.history()
    assert [s for s, _ in hist] == [0, 1]
    assert hist[1][1] == {"rollout/tokens": 15.0, "train/loss": 2.0}
    svc.close()   # flushes step 2
    lines = [json.loads(l) for l in open(path)]
    assert [l["step"] for l in lines] == [0, 1, 2]


def test_http_front_and_client_roundtrip():
    svc = MetricsService()
    srv, url = serve(svc)
    try:
        c = MetricsClient(url=url)
        c.log_metric(3, "x", 1.5)
        c.log_metrics_batch(3, {"y": 2, "z": 3})
        c.log_error("rollout", "engine 2 lost", step=3)
        c.report_step(3)
        assert svc.history() == [(3, {"x": 1.5, "y": 2.0, "z": 3.0})]
        assert svc.errors()[0]["source"] == "rollout"
    finally:
        srv.shutdown()


def test_flops_counter_matches_hand_count():
    cfg = get_config("qwen3-8b")
    lens = [2560, 2560]
    f = forward_flops(cfg, lens)
    T, h, L = 5120, 4096, 36
    proj = L * 2 * T * h * (32 * 128 * 2 + 2 * 8 * 128)
    core = L * 4 * (2 * 2560 ** 2) * 32 * 128 * 0.5
    mlp = L * 2 * T * h * 12288 * 3
    head = 2 * T * h * 151936
    assert abs(f.total - (proj + core + mlp + head)) / f.total < 1e-12
    step = train_step_flops(cfg, lens, forward_only_passes=2)
    assert abs(step / f.total - 5.0) < 1e-12
    assert 0 < mfu(step, 0.6, 1, 2250.0) < 1
    moe = get_config("qwen3-30b-a3b")
    fm = forward_flops(moe, [1024])
    assert fm.router > 0 and fm.mlp == moe.num_layers * 2 * 1024 * moe.hidden_size * moe.moe_ffn_hidden_size * 3 * moe.moe_top_k


def test_profiler_window_writes_trace(tmp_path):
    p = TrainProfiler(str(tmp_path), start_step=1, end_step=3)
    for _ in range(5):
        torch.randn(64, 64) @ torch.randn(64, 64)
        p.step()
    p.close()
    assert p.trace_path and os.path.getsize(p.trace_path) > 0
    off = TrainProfiler(None)
    off.step()
    assert not off.enabled
