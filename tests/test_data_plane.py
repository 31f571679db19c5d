import threading
import time

import pytest

from relax_b200.data import transfer_queue as tq
from relax_b200.data.samplers import IdentityWindowSampler, SeqlenBalancedSampler, StreamingTokenBudgetSampler
from relax_b200.data.seqlen_balancing import balanced_microbatches, first_fit_decreasing, karmarkar_karp


def test_per_task_consumption_and_column_writeback():
    q = tq.TransferQueue()
    q.put({"tokens": [[1], [2], [3]]}, "train_0", custom_meta=[{"total_lengths": 1}] * 3)
    m = q.get_meta(["tokens"], 2, "train_0", "actor_fwd")
    assert m.row_ids == [0, 1] and q.get_data(m)["tokens"] == [[1], [2]]
    # the actor needs log_probs, which actor_fwd writes back later
    assert q.get_meta(["tokens", "log_probs"], 2, "train_0", "actor", timeout=0.05) is None
    q.put({"log_probs": [[-1.0], [-2.0]]}, "train_0", row_ids=m.row_ids)
    m2 = q.get_meta(["tokens", "log_probs"], 2, "train_0", "actor")
    assert q.get_data(m2)["log_probs"] == [[-1.0], [-2.0]]
    # each task sees each row once
    m3 = q.get_meta(["tokens"], 1, "train_0", "actor_fwd")
    assert m3.row_ids == [2]
    q.seal("train_0")
    assert q.check_consumption_status("actor_fwd", "train_0")
    assert not q.check_consumption_status("actor", "train_0")
    assert not q.check_production_status(["log_probs"], "train_0")
    q.reset_consumption("train_0", "actor_fwd")
    assert q.get_meta(["tokens"], None, "train_0", "actor_fwd").row_ids == [0, 1, 2]


def test_blocking_get_wakes_on_put_and_partial_final_batch():
    q = tq.TransferQueue()
    out = {}

    def consumer():
        out["m"] = q.get_meta(["x"], 4, "p", "t", timeout=5, allow_partial=True)

    th = threading.Thread(target=consumer)
    th.start()
    time.sleep(0.05)
    q.put({"x": [1, 2, 3]}, "p", is_last=True)
    th.join(5)
    assert out["m"].row_ids == [0, 1, 2]
    assert q.check_stream_drained("t", "p", ["x"])
    assert q.get_meta(["x"], 4, "p", "t", timeout=0.05) is None


def test_capacity_and_partition_listing():
    q = tq.TransferQueue(capacity_partitions=2)
    q.put({"x": [1]}, "train_0")
    q.put({"x": [1]}, "train_1")
    with pytest.raises(RuntimeError):
        q.put({"x": [1]}, "train_2")
    q.clear_partition("train_0")
    q.put({"x": [1]}, "train_2")
    assert q.get_partition_list() == ["train_1", "train_2"]
    assert tq.partition_rollout_id("train_12") == 12 and tq.partition_name(3) == "train_3"


def test_karmarkar_karp_balance():
    lens = [100, 90, 80, 20, 20, 10, 5, 5]
    bins = karmarkar_karp(lens, 2)
    sums = [sum(lens[i] for i in b) for b in bins]
    assert sorted(i for b in bins for i in b) == list(range(8)) and abs(sums[0] - sums[1]) <= 10
    bins = karmarkar_karp(lens, 4, equal_size=True)
    assert all(len(b) == 2 for b in bins)
    with pytest.raises(ValueError):
        karmarkar_karp(lens[:7], 2, equal_size=True)


def test_token_cap_microbatches():
    lens = [60, 50, 40, 30, 20, 10]
    ffd = first_fit_decreasing(lens, 100)
    assert all(sum(lens[i] for i in b) <= 100 for b in ffd)
    mbs = balanced_microbatches(lens, 100)
    assert sorted(i for b in mbs for i in b) == list(range(6))
    assert all(sum(lens[i] for i in b) <= 100 for b in mbs)
    assert len(balanced_microbatches(lens, 100, multiple_of=4)) % 4 == 0


def test_samplers():
    ready = list(range(8))
    meta = [{"total_lengths": l, "sample_index": i // 2} for i, l in enumerate([10, 90, 20, 80, 30, 70, 40, 60])]
    a = SeqlenBalancedSampler(0, 2)(ready, meta, 4)
    b = SeqlenBalancedSampler(1, 2)(ready, meta, 4)
    assert sorted(a + b) == ready and len(a) == len(b) == 4
    ta, tb = sum(meta[i]["total_lengths"] for i in a), sum(meta[i]["total_lengths"] for i in b)
    assert abs(ta - tb) <= 20
    assert StreamingTokenBudgetSampler(100)(ready, meta, None) == [0, 1]
    s = IdentityWindowSampler(max_tokens=250, window_samples=2)
    assert s(ready, meta, None) == [0, 1, 2, 3]          # both rows of samples 0 and 1, never split
    s.advance_window()
    assert s(ready, meta, None) == [4, 5, 6, 7]


def test_log_rollout_data_masked_token_means_and_scalars():
    import torch

    from relax_b200.data.rollout_log import log_rollout_data

    batch = {"tokens": [[1, 2, 3, 4], [5, 6, 7]], "response_lengths": [2, 2], "total_lengths": [4, 3],
             "loss_masks": [[1.0, 0.0], [1.0, 1.0]], "rewards": [1.0, 0.0], "raw_reward": [2.0, 4.0],
             "log_probs": [torch.tensor([-1.0, -9.0]), torch.tensor([-2.0, -4.0])], "advantages": [[0.5, 0.5], [-0.5, -0.5]]}
    m = log_rollout_data(batch)
    assert m["rollout/rewards"] == 0.5 and m["rollout/raw_reward"] == 3.0 and m["rollout/response_lengths"] == 2.0
    assert m["rollout/prompt_lengths"] == 1.5
    assert abs(m["rollout/log_probs"] - (-1.0 + -3.0) / 2) < 1e-6        # the masked-out -9 does not count
    assert abs(m["rollout/advantages"]) < 1e-9 and "rollout/tokens" not in m


def test_streaming_iterator_consumes_while_the_producer_is_still_writing():
    """StreamingTQIterator: token-budget micro-batches arrive while rows are still being produced, data-parallel ranks
    get disjoint rows, the loss scale rides along, and iteration ends when the sealed partition is consumed."""
    import threading
    import time

    from relax_b200.data import transfer_queue as tq
    from relax_b200.data.samplers import StreamingTQIterator

    q = tq.TransferQueue()
    part = tq.partition_name(0)
    lens = [5, 9, 4, 7, 6, 3, 8, 2]

    def produce():
        for i, L in enumerate(lens):
            time.sleep(0.02)
            q.put({"tokens": [list(range(L))], "response_lengths": [L // 2]}, part, custom_meta=[{"total_lengths": L, "sample_index": i}],
                  is_last=(i == len(lens) - 1))

    th = threading.Thread(target=produce)
    th.start()
    seen = {0: [], 1: []}
    first_batch_time = {}

    def consume(r):
        it = StreamingTQIterator(q, ["tokens", "response_lengths"], part, token_budget=12, loss_scale=0.5, dp_rank=r, dp_size=2)
        for batch, meta in it:
            first_batch_time.setdefault(r, time.monotonic())
            assert batch["__loss_scale__"] == 0.5
            assert sum(len(t) for t in batch["tokens"]) <= 12 or len(batch["tokens"]) == 1
            seen[r] += [len(t) for t in batch["tokens"]]

    cs = [threading.Thread(target=consume, args=(r,)) for r in (0, 1)]
    [c.start() for c in cs]
    th.join()
    t_done = time.monotonic()
    [c.join(timeout=20) for c in cs]
    assert sorted(seen[0]) == sorted(lens[0::2]) and sorted(seen[1]) == sorted(lens[1::2])
    assert min(first_batch_time.values()) < t_done, "consumption started before the producer finished"
