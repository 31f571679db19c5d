"""Fully-asynchronous and hybrid execution: roles as concurrent loops around the
data plane, bounded staleness, gated weight updates.

Reference behaviour: rollout loop with staleness gate and peer barrier
(relax/components/rollout.py:403-523), forward-only roles that add columns
(relax/components/actor_fwd.py:38-49, relax/backends/megatron/actor.py:1098-1191),
CPU advantages service (relax/components/advantages.py:55-232), actor loop that
waits for data, trains, asks the rollout for permission and pushes weights
(relax/components/actor.py:192-321, relax/backends/megatron/actor.py:1569-1691,
1824-1959), heartbeats (relax/core/service.py:112-129).

Each role is a ``RoleLoop`` (a thread here; on a multi-GPU job one instance per
member rank).  Roles only talk through the data plane (rows and columns of
partition ``train_{rollout_id}``), the weight channel and the health registry,
so the same loops serve the threaded single-process mode used in tests and the
rank-subset SPMD mode.
"""
from __future__ import annotations

import threading
import time
import traceback
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from ..algo import loss as L
from ..algo.ppo_utils import Segments
from ..data import transfer_queue as tq
from ..data.convert import convert_samples_to_train_data, custom_meta_rows
from ..health.monitor import HealthRegistry
from .registry import Role, process_role, satisfy_staleness


@dataclass
class PipelineConfig:
    num_rollout: int = 4
    max_staleness: int = 1
    rollout_batch_size: int = 4
    fully_async: bool = True
    hybrid: bool = False
    true_on_policy_mode: bool = False
    advantage_estimator: str = "grpo"
    update_weights_interval: int = 1
    poll_interval: float = 0.005
    debug_rollout_only: bool = False
    debug_train_only: bool = False
    loss_type: str = "policy_loss"
    stream_batch_rows: Optional[int] = None   # rows a consumer asks for at once (None = whole partition)


class WeightChannel:
    """Trainer -> consumers weight hand-off with versioning and a rollout-side gate.

    ``request_update`` is the trainer's ``/can_do_update_weight_for_async`` call: it
    returns once the rollout loop has parked at a safe point; ``end_update`` releases
    it (``/end_update_weight``).  Forward-only roles poll :meth:`wait_version`."""

    def __init__(self):
        self._cv = threading.Condition()
        self.version = 0
        self._want_update = False
        self._rollout_parked = False
        self.lock = threading.Lock()      # mutual exclusion of weight syncs (the reference's Lock actor)
        self.payload = None

    # trainer side
    def request_update(self, timeout: float = 60.0) -> bool:
        with self._cv:
            self._want_update = True
            self._cv.notify_all()
            ok = self._cv.wait_for(lambda: self._rollout_parked or self._rollout_absent, timeout)
            return ok

    _rollout_absent = False

    def publish(self, payload, version: int):
        with self._cv:
            self.payload, self.version = payload, version
            self._cv.notify_all()

    def end_update(self):
        with self._cv:
            self._want_update = False
            self._cv.notify_all()

    # rollout side: called between generation steps
    def park_if_requested(self):
        with self._cv:
            if not self._want_update:
                return
            self._rollout_parked = True
            self._cv.notify_all()
            self._cv.wait_for(lambda: not self._want_update)
            self._rollout_parked = False

    def mark_rollout_absent(self):
        with self._cv:
            self._rollout_absent = True
            self._cv.notify_all()

    def wait_version(self, v: int, timeout: float = 60.0):
        with self._cv:
            self._cv.wait_for(lambda: self.version >= v, timeout)
            return self.version, self.payload


class RoleLoop(threading.Thread):
    role: Role

    def __init__(self, pipe: "AsyncPipeline"):
        super().__init__(daemon=True, name=f"role-{self.role.value}")
        self.pipe = pipe
        self.step = 0
        self.error: Optional[str] = None
        self.stop_flag = threading.Event()

    def beat(self):
        self.pipe.health.heartbeat(self.role.value, step=self.step)

    def run(self):
        try:
            self.loop()
        except Exception as e:  # noqa: BLE001
            self.error = traceback.format_exc()
            self.pipe.health.report_error(self.role.value, repr(e))

    def loop(self):
        raise NotImplementedError


class RolloutLoop(RoleLoop):
    role = Role.rollout

    def loop(self):
        p, cfg = self.pipe, self.pipe.cfg
        for rid in range(p.start_rollout_id, cfg.num_rollout):
            # bounded staleness: do not run more than max_staleness ahead of the oldest unconsumed partition
            while not satisfy_staleness(p.queue.get_partition_list(), rid - 1, cfg.max_staleness):
                if self.stop_flag.is_set():
                    return
                p.weights.park_if_requested()
                self.beat()
                time.sleep(cfg.poll_interval)
            p.weights.park_if_requested()
            samples = p.generate_fn(rid)
            p.rollout_started.append((rid, p.weights.version, list(p.queue.get_partition_list())))
            batch = p.convert_fn(samples)
            p.queue.put(batch, tq.partition_name(rid), custom_meta=custom_meta_rows(batch), is_last=True)
            self.step = rid + 1
            self.beat()
        p.weights.mark_rollout_absent()


class ForwardLoop(RoleLoop):
    """actor_fwd / reference: add a log-prob column to every row, follow weight versions."""

    def __init__(self, pipe, role: Role, column: str, compute: Callable, follows_weights: bool):
        self.role = role
        super().__init__(pipe)
        self.column, self.compute, self.follows_weights = column, compute, follows_weights
        self.seen_version = 0

    def loop(self):
        p, cfg = self.pipe, self.pipe.cfg
        for rid in range(p.start_rollout_id, cfg.num_rollout):
            part = tq.partition_name(rid)
            while not self.stop_flag.is_set():
                meta = p.queue.get_meta(["tokens", "response_lengths"], cfg.stream_batch_rows, part, self.role.value,
                                        timeout=0.05, allow_partial=True)
                if meta is None:
                    if p.queue.check_consumption_status(self.role.value, part):
                        break
                    self.beat()
                    continue
                data = p.queue.get_data(meta)
                out = self.compute(data)
                p.queue.put({self.column: [x.detach().cpu().tolist() for x in out]}, part, row_ids=meta.row_ids)
                self.beat()
            if self.follows_weights:
                v, payload = p.weights.wait_version(self.seen_version + 1, timeout=0.0)
                if v > self.seen_version and payload is not None:
                    p.recv_weight_fn(self.role, payload)
                    self.seen_version = v
            self.step = rid + 1


class AdvantagesLoop(RoleLoop):
    role = Role.advantages

    def loop(self):
        p, cfg = self.pipe, self.pipe.cfg
        need = ["rewards", "response_lengths", "loss_masks"]
        if p.needs_old_logp:
            need.append("log_probs")
        if p.needs_ref:
            need.append("ref_log_probs")
        for rid in range(p.start_rollout_id, cfg.num_rollout):
            part = tq.partition_name(rid)
            while not self.stop_flag.is_set():
                meta = p.queue.get_meta(need, cfg.stream_batch_rows, part, self.role.value, timeout=0.05, allow_partial=True)
                if meta is None:
                    if p.queue.check_consumption_status(self.role.value, part):
                        break
                    self.beat()
                    continue
                d = p.queue.get_data(meta)
                seg = Segments.from_lengths(d["response_lengths"])
                cat = lambda k: torch.cat([torch.tensor(x, dtype=torch.float32) for x in d[k]]) if k in d else None
                adv, ret = L.compute_advantages_and_returns(
                    cfg.advantage_estimator, torch.tensor(d["rewards"]), seg, cat("loss_masks"),
                    log_probs=cat("log_probs"), ref_log_probs=cat("ref_log_probs"), kl_coef=p.kl_coef)
                p.queue.put({"advantages": [a.tolist() for a in seg.split(adv)], "returns": [a.tolist() for a in seg.split(ret)]},
                            part, row_ids=meta.row_ids)
                self.beat()
            self.step = rid + 1


class ActorLoop(RoleLoop):
    role = Role.actor

    def loop(self):
        p, cfg = self.pipe, self.pipe.cfg
        need = ["tokens", "response_lengths", "rewards", "loss_masks", "total_lengths", "sample_index_mask_sums"]
        need += p.actor_extra_fields
        for rid in range(p.start_rollout_id, cfg.num_rollout):
            part = tq.partition_name(rid)
            rows = []
            while not self.stop_flag.is_set():
                meta = p.queue.get_meta(need, cfg.stream_batch_rows, part, self.role.value, timeout=0.05, allow_partial=True)
                if meta is None:
                    if p.queue.check_consumption_status(self.role.value, part):
                        break
                    self.beat()
                    continue
                rows.append(p.queue.get_data(meta))
                self.beat()
            if self.stop_flag.is_set():
                return
            data = {k: [x for r in rows for x in r[k]] for k in rows[0]} if rows else None
            if data is not None:
                metrics = p.train_fn(rid, data)
                p.metrics.append((rid, metrics))
            p.queue.clear_partition(part)
            self.step = rid + 1
            if (rid + 1) % cfg.update_weights_interval == 0:
                with p.weights.lock:
                    if p.weights.request_update():
                        payload = p.export_weights_fn()
                        p.push_to_rollout_fn(payload)
                        p.weights.publish(payload, self.step)
                    p.weights.end_update()
            self.beat()


class AsyncPipeline:
    """Wires role loops to user-supplied compute callbacks.

    Callbacks: ``generate_fn(rollout_id) -> samples``, ``convert_fn(samples) -> batch``,
    ``train_fn(rollout_id, batch) -> metrics``, ``export_weights_fn() -> payload``,
    ``push_to_rollout_fn(payload)``, ``recv_weight_fn(role, payload)``,
    ``fwd_fn(batch) -> list[tensor]`` (old-policy log-probs), ``ref_fn(batch)``."""

    def __init__(self, cfg: PipelineConfig, *, generate_fn, convert_fn, train_fn, export_weights_fn,
                 push_to_rollout_fn, recv_weight_fn=None, fwd_fn=None, ref_fn=None, kl_coef: float = 0.0,
                 start_rollout_id: int = 0, queue: Optional[tq.TransferQueue] = None):
        self.cfg = cfg
        self.queue = queue or tq.TransferQueue(capacity_partitions=cfg.max_staleness + 2)
        self.weights = WeightChannel()
        self.health = HealthRegistry(heartbeat_timeout=120.0)
        self.generate_fn, self.convert_fn, self.train_fn = generate_fn, convert_fn, train_fn
        self.export_weights_fn, self.push_to_rollout_fn = export_weights_fn, push_to_rollout_fn
        self.recv_weight_fn = recv_weight_fn or (lambda role, payload: None)
        self.kl_coef = kl_coef
        self.start_rollout_id = start_rollout_id
        self.metrics: list = []
        self.rollout_started: list = []
        roles = process_role(cfg)
        self.roles = roles
        inline_forward = cfg.hybrid or not cfg.fully_async
        self.needs_old_logp = Role.actor_fwd in roles and fwd_fn is not None
        self.needs_ref = Role.reference in roles and ref_fn is not None and not inline_forward
        self.actor_extra_fields = []
        self.loops: list[RoleLoop] = []
        if Role.rollout in roles:
            self.loops.append(RolloutLoop(self))
        if not inline_forward:
            if self.needs_old_logp:
                self.loops.append(ForwardLoop(self, Role.actor_fwd, "log_probs", fwd_fn, follows_weights=True))
                self.actor_extra_fields.append("log_probs")
            if self.needs_ref:
                self.loops.append(ForwardLoop(self, Role.reference, "ref_log_probs", ref_fn, follows_weights=False))
                self.actor_extra_fields.append("ref_log_probs")
            if Role.advantages in roles:
                self.loops.append(AdvantagesLoop(self))
                self.actor_extra_fields += ["advantages", "returns"]
        if Role.actor in roles:
            self.loops.append(ActorLoop(self))
        if Role.rollout not in roles:
            self.weights.mark_rollout_absent()

    def run(self, timeout: float = 600.0):
        for l in self.loops:
            l.start()
        deadline = time.monotonic() + timeout
        for l in self.loops:
            l.join(max(0.0, deadline - time.monotonic()))
        errs = [f"{l.role.value}: {l.error}" for l in self.loops if l.error]
        alive = [l.role.value for l in self.loops if l.is_alive()]
        if alive:
            for l in self.loops:
                l.stop_flag.set()
            raise TimeoutError(f"roles still running after {timeout}s: {alive}")
        if errs:
            raise RuntimeError("role failure:\n" + "\n".join(errs))
        return self.metrics

    def stop(self):
        for l in self.loops:
            l.stop_flag.set()
