"""DCS: topology / global ranks, weight-metadata long-poll, tensor fusion, bucketed broadcast between processes."""
import threading
import time

import torch

from relax_b200.weight_sync.dcs import (Coordinator, CoordinatorClient, DeviceDirectBackend, TensorFusion, TopologyManager,
                                         serve)
from tests._mp import run_distributed


def test_topology_orders_roles_and_builds_update_groups():
    t = [0.0]
    topo = TopologyManager(heartbeat_timeout_s=10, clock=lambda: t[0])
    topo.register("rollout", 0)
    topo.register("actor", 1, meta={"pp_rank": 1, "tp_rank": 0})
    topo.register("actor", 0, meta={"pp_rank": 0, "tp_rank": 0})
    topo.register("actor_fwd", 0)
    topo.register("reference", 0)
    assert [topo.global_rank(*k) for k in [("actor", 0), ("actor", 1), ("actor_fwd", 0), ("reference", 0), ("rollout", 0)]] == [0, 1, 2, 3, 4]
    g = topo.update_group_ranks(pp_size=2)
    assert g == {"update_actor_pp_0": [0, 2, 3, 4], "update_actor_pp_1": [1, 2, 3, 4]}
    t[0] = 11
    assert not topo.alive("rollout", 0)
    assert topo.heartbeat("rollout", 0) and topo.alive("rollout", 0)
    topo.unregister("actor_fwd", 0)
    assert topo.global_rank("reference", 0) == 2


def test_weight_meta_long_poll_over_http():
    coord = Coordinator()
    srv, url = serve(coord)
    try:
        c = CoordinatorClient(url)
        assert c.register("actor", 0) == 0 and c.register("rollout", 0) == 1
        assert c.recv_weight_meta(-1, timeout_s=0.2) is None
        got = {}

        def waiter():
            got["msg"] = c.recv_weight_meta(-1, timeout_s=10)

        th = threading.Thread(target=waiter)
        th.start()
        time.sleep(0.2)
        CoordinatorClient(url).send_weight_meta(5, {"buckets": []})
        th.join(5)
        assert got["msg"]["version"] == 5
        assert c.recv_weight_meta(5, timeout_s=0.2) is None   # nothing newer
    finally:
        srv.shutdown()


def test_tensor_fusion_roundtrip_and_bucket_limit():
    torch.manual_seed(0)
    named = [(f"w{i}", torch.randn(64, 64)) for i in range(5)] + [("b", torch.randn(7).bfloat16())]
    f = TensorFusion(bucket_bytes=2 * 64 * 64 * 4)
    plan = f.plan(named)
    assert len(plan) == 4 and {l.dtype for l in plan} == {"torch.float32", "torch.bfloat16"}
    tens = dict(named)
    for lay in plan:
        buf = f.pack(lay, tens, "cpu")
        for n, t in f.unpack(lay, buf):
            assert torch.equal(t, tens[n])


def _bcast_worker(rank, world, url):
    client = CoordinatorClient(url)
    client.register("actor" if rank == 0 else "rollout", 0)
    be = DeviceDirectBackend(client, src=0, bucket_bytes=40000)
    g = torch.Generator().manual_seed(1)
    named = [(f"layer{i}.w", torch.randn(50, 60, generator=g)) for i in range(4)]
    if rank == 0:
        n = be.update_weights(named, version=3)
        return n
    got = {}
    v = be.recv_weight(lambda name, t: got.__setitem__(name, t.clone()), timeout_s=30)
    ok = v == 3 and all(torch.equal(got[n], t) for n, t in named)
    return ok


def test_bucketed_broadcast_between_processes():
    coord = Coordinator()
    srv, url = serve(coord)
    try:
        out = run_distributed(_bcast_worker, 2, url)
        assert out[0] == 2 and out[1] is True
    finally:
        srv.shutdown()
