"""TransferQueue over TCP: producer and consumers in different processes, async client calls, pinned pool reuse."""
import asyncio

import torch

from relax_b200.data.tq_service import PinnedPool, TQClient, TQServer
from tests._mp import run_distributed


def _rows(n, base=0):
    return {"tokens": [torch.arange(5 + i) + base for i in range(n)], "rewards": [float(i) for i in range(n)]}


def test_roundtrip_and_per_task_consumption():
    srv = TQServer()
    try:
        c = TQClient(srv.address, PinnedPool(pin=False))
        c.put(_rows(4), "train_0", is_last=True)
        assert c.get_partition_list() == ["train_0"] and c.num_rows("train_0") == 4
        m = c.get_meta(["tokens", "rewards"], 3, "train_0", "actor")
        d = c.get_data(m)
        assert len(d["tokens"]) == 3 and torch.equal(d["tokens"][1], torch.arange(6)) and d["rewards"][2] == 2.0
        m2 = c.get_meta(["tokens"], None, "train_0", "reference")      # another task sees every row again
        assert len(m2) == 4
        assert not c.check_consumption_status("actor", "train_0")
        c.get_data(c.get_meta(["tokens"], None, "train_0", "actor"))
        assert c.check_consumption_status("actor", "train_0")
        assert c.get_meta(["nope"], 1, "missing", "actor", timeout=0.1) is None   # waits, then gives up
        try:
            c._call("no_such_method")
            assert False
        except RuntimeError:
            pass                                                                  # server-side errors come back as errors
        # pooled buffers are reused once released
        pool = c.pool
        b = pool.take(1000)
        pool.give(b)
        assert pool.take(900) is b and pool.reuses >= 1

        async def go():
            await c.async_put(_rows(2, 100), "train_1", is_last=True)
            mm = await c.async_get_meta(["tokens"], None, "train_1", "actor")
            return await c.async_get_data(mm)

        out = asyncio.run(go())
        assert torch.equal(out["tokens"][0], torch.arange(5) + 100)
        c.clear_partition("train_0")
        assert c.get_partition_list() == ["train_1"]
        c.close()
    finally:
        srv.close()


def _proc(rank, world, address):
    c = TQClient(address, PinnedPool(pin=False))
    if rank == 0:
        for rid in range(3):
            c.put(_rows(4, 10 * rid), f"train_{rid}", is_last=True)
        return "produced"
    got = []
    import time

    for rid in range(3):
        part = f"train_{rid}"
        t0 = time.time()
        while part not in c.get_partition_list() or not c.check_production_status(["tokens"], part):
            time.sleep(0.01)
            assert time.time() - t0 < 30
        d = c.get_data(c.get_meta(["tokens"], None, part, f"consumer{rank}"))
        got.append(int(d["tokens"][0][0]))
    return got


def test_producer_and_consumers_in_other_processes():
    srv = TQServer()
    try:
        out = run_distributed(_proc, 3, srv.address)
        assert out[0] == "produced" and out[1] == [0, 10, 20] and out[2] == [0, 10, 20]
    finally:
        srv.close()
