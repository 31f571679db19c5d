"""Fully-asynchronous / hybrid RL on DISJOINT GPU pools: trainer ranks and rollout ranks are different processes.

The reference places roles on GPU pools from ``--resource`` (relax/core/controller.py:606-763), streams rollout
batches to the trainer through TransferQueue, bounds how far generation may run ahead of training
(relax/components/rollout.py:298-315) and pushes new weights from the trainer to the engines while they pause at a
safe point (relax/backends/megatron/actor.py:1569-1691, 1931-1968; relax/distributed/checkpoint_service/backends/
device_direct.py:598-778).  The same job here, in SPMD form:

* ``assign_ranks`` turns ``--resource`` into rank lists; every process builds one :class:`DisaggregatedRL`, which
  creates the trainer's parallel groups over the trainer ranks and one tensor-parallel group per rollout engine;
* **data plane**: the first trainer rank hosts the queue service (:mod:`relax_b200.data.tq_service`); the leader of
  each engine puts its rows into partition ``train_{rollout_id}``, the trainer's fetcher takes the sealed partition
  and hands every data-parallel replica its share;
* **staleness gate**: a rollout step starts only while it is at most ``max_staleness`` ahead of the oldest
  partition the trainer has not consumed;
* **weight push**: after a training step the trainer raises ``wsync/request`` in the job's key-value store; rollout
  ranks look at it between decode windows (a safe point: nothing that reads the weights is in flight), answer
  ``ready``, and the trainer ranks store their shards directly into the engines' parameter buffers over NVLink
  (:class:`~relax_b200.weight_sync.peer_push.PeerWeightPusher`), then post ``done`` with the new version; generation
  continues with the new weights and tags its tokens with the version.  ``weight_push="broadcast"`` runs the
  NCCL-broadcast arm of the same plan instead (the A/B baseline);
* the reference / old-policy log-probs are computed inside the trainer by switching weight tags (hybrid mode's
  in-process forward roles).

Every wait on another pool is bounded by ``handshake_timeout_s`` and raises on expiry.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist

from ..data import transfer_queue as tq
from ..data.convert import convert_samples_to_train_data, custom_meta_rows
from ..data.tq_service import TQClient, TQServer
from ..models.config import ModelConfig, get_config
from ..parallel.state import GroupInfo, ParallelDims, init_parallel_state
from ..rewards import get_reward_spec
from ..rollout.data_source import RolloutDataSource, SyntheticPromptDataset
from ..rollout.engine import RolloutEngine, SamplingParams
from ..train.actor import TrainActor, TrainConfig
from ..types import SampleStatus
from ..weight_sync.peer_push import BroadcastPusher, PeerWeightPusher, SharedWeightRegion
from ..weight_sync.plan import TrainerLayout
from .registry import satisfy_staleness


@dataclass
class DisaggConfig:
    model: ModelConfig = field(default_factory=lambda: get_config("tiny"))
    train: TrainConfig = field(default_factory=TrainConfig)
    trainer_ranks: tuple = (0,)
    rollout_ranks: tuple = (1,)
    trainer_tp: int = 1
    rollout_tp: int = 1
    rollout_batch_size: int = 8          # prompts per rollout step, all engines together
    prompt_len: int = 64
    max_response_len: int = 64
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    rm_type: str = "parity"
    eos_token_id: Optional[int] = None
    kv_blocks: int = 512
    kv_block_size: int = 16
    max_running: int = 256
    use_cuda_graph: bool = True
    num_rollout: int = 4
    max_staleness: int = 1
    update_weights_interval: int = 1
    speculative: bool = False             # the engines draft with the model's MTP block (its weights are pushed with the rest)
    speculative_steps: int = 1
    num_iters_per_train_update: int = 1   # > 1: the engines publish finished prompt groups in that many parts per rollout
                                          # and the trainer runs its forward-only passes on each part as it arrives
    image_grid_side: int = 0              # vision-language models: patches per side of the synthetic images (0: 4 x merge size)
    weight_push: str = "peer"            # "peer": NVLink stores into the engines' buffers; "broadcast": NCCL baseline
    seed: int = 0
    rollout_seed: int = 42
    num_prompts: int = 1 << 14
    poll_interval: float = 0.002
    handshake_timeout_s: float = 300.0
    tag: Optional[str] = None            # names the Unix sockets of this job (default: the rendezvous port)


class _Store:
    """Counters and flags of the job in the rendezvous key-value store (host side only)."""

    def __init__(self, prefix: str):
        from torch.distributed import distributed_c10d as c10d

        self.s, self.prefix = c10d._get_default_store(), prefix

    def add(self, key: str, delta: int = 0) -> int:
        return int(self.s.add(self.prefix + key, int(delta)))

    def set(self, key: str, value: str):
        self.s.set(self.prefix + key, value)

    def get(self, key: str) -> str:
        return self.s.get(self.prefix + key).decode()

    def wait_ge(self, key: str, target: int, timeout: float, poll: float, what: str):
        deadline = time.monotonic() + timeout
        while self.add(key, 0) < target:
            if time.monotonic() > deadline:
                raise TimeoutError(f"{what}: {key} stayed below {target} for {timeout:.0f} s")
            time.sleep(poll)


class DisaggregatedRL:
    def __init__(self, cfg: DisaggConfig, device="cpu"):
        if not dist.is_initialized():
            raise RuntimeError("disjoint trainer / rollout pools need torch.distributed (one process per rank)")
        self.cfg = cfg
        self.device = torch.device(device)
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        tr, ro = tuple(cfg.trainer_ranks), tuple(cfg.rollout_ranks)
        if set(tr) & set(ro):
            raise ValueError("trainer and rollout pools must be disjoint (use the colocated runner to share GPUs)")
        if len(ro) % cfg.rollout_tp or len(tr) % cfg.trainer_tp:
            raise ValueError("pool sizes must be multiples of the tensor-parallel sizes")
        self.is_trainer, self.is_rollout = self.rank in tr, self.rank in ro
        self.tag = cfg.tag or os.environ.get("MASTER_PORT", "0")
        self.store = _Store(f"disagg{self.tag}/")
        # ---- groups: creation is collective over ALL ranks of the job
        dims = ParallelDims(tp=cfg.trainer_tp, dp=len(tr) // cfg.trainer_tp)
        self.ps = init_parallel_state(dims, role_ranks=tr)
        rtp = cfg.rollout_tp
        self.engines = [ro[i:i + rtp] for i in range(0, len(ro), rtp)]
        self.engine_id, eng_group = -1, None
        for i, e in enumerate(self.engines):
            g = dist.new_group(list(e)) if rtp > 1 else None
            if self.rank in e:
                self.engine_id, eng_group = i, g
        self.bcast_groups = []
        if cfg.weight_push == "broadcast":
            for s in tr[:cfg.trainer_tp]:          # replica 0 is the source of every engine
                self.bcast_groups.append(dist.new_group([s] + list(ro)))
        # ---- data plane
        self.tq_server = None
        if self.rank == tr[0]:
            self.tq_server = TQServer(tq.TransferQueue(capacity_partitions=cfg.max_staleness + 2))
            self.store.set("tq_addr", f"{self.tq_server.address[0]}:{self.tq_server.address[1]}")
        self.is_fetcher = self.rank == tr[0]
        self.is_leader = self.is_rollout and self.rank == self.engines[self.engine_id][0]
        self.tq = None
        if self.is_fetcher or self.is_leader:
            host, port = self.store.get("tq_addr").rsplit(":", 1)
            self.tq = TQClient((host, int(port)))
        # ---- roles
        dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[cfg.model.dtype]
        self.actor = self.engine = self.region = self.pusher = self.bcast = None
        self.applied_version = -1
        if self.is_trainer:
            need_ref = cfg.train.loss.use_kl_loss or cfg.train.kl_coef != 0
            self.actor = TrainActor(cfg.model, cfg.train, self.ps, device=device, seed=cfg.seed, with_reference=need_ref)
            if cfg.model.vision is not None and any(p.requires_grad for p in self.actor.model.vision.parameters()):
                raise ValueError("disaggregated mode pushes the language model's weights only: freeze the vision tower "
                                 "(--freeze-vision-model / freeze_params_name_list=['^vision\\.'])")
        if self.is_rollout:
            cuda = self.device.type == "cuda"
            shm = None if cuda else f"/dev/shm/relax_b200_{self.tag}_{self.rank}.bin"
            self.engine = RolloutEngine(cfg.model, GroupInfo(eng_group, tuple(self.engines[self.engine_id]),
                                                             self.engines[self.engine_id].index(self.rank)),
                                        device=device, dtype=dtype, num_kv_blocks=cfg.kv_blocks, block_size=cfg.kv_block_size,
                                        max_running=cfg.max_running, seed=cfg.rollout_seed + self.engine_id,
                                        use_cuda_graph=cfg.use_cuda_graph, memory_saver=True if cuda else False,
                                        max_model_len=cfg.prompt_len + cfg.max_response_len, eos_token_id=cfg.eos_token_id,
                                        weights_shared_path=shm, speculative=cfg.speculative, speculative_steps=cfg.speculative_steps)
            self._shm = shm
            if cfg.weight_push == "peer":
                self.region = SharedWeightRegion(self.engine.weights, self.tag, self.rank)
            if cfg.model.vision is not None:
                # vision-language: the rollout rank builds the tower itself with the trainer's initialisation (same seed
                # rule as TrainActor) and keeps it; the trainer side must therefore hold the tower fixed (checked there)
                from ..models.vision import VisionEncoder, vision_config_from_model
                from ..rollout.data_source import SyntheticImagePromptDataset

                self.vision = VisionEncoder(vision_config_from_model(cfg.model), dtype=dtype, device=device, seed=cfg.seed + 17)
                self.engine.attach_vision(self.vision)
                v = cfg.model.vision
                side = cfg.image_grid_side or 4 * v.spatial_merge_size
                n_img = side * side // v.spatial_merge_size ** 2
                ds = SyntheticImagePromptDataset(cfg.num_prompts, max(1, (cfg.prompt_len - n_img) // 2), cfg.model.vocab_size,
                                                 cfg.model.image_token_id, (side, side),
                                                 v.in_channels * v.temporal_patch_size * v.patch_size ** 2, v.spatial_merge_size, seed=cfg.seed)
            else:
                ds = SyntheticPromptDataset(cfg.num_prompts, cfg.prompt_len, cfg.model.vocab_size, seed=cfg.seed)
            self.data_source = RolloutDataSource(ds, cfg.train.n_samples_per_prompt, shuffle=False, seed=cfg.rollout_seed)
            self.reward_fn = get_reward_spec(cfg.rm_type).fn
        dist.barrier()        # every exported buffer is being served before anyone maps it
        if self.is_trainer:
            dp, my_dp = self.ps.dp.size, self.ps.dp.rank
            mine = [e for i, e in enumerate(self.engines) if i % dp == my_dp]
            if cfg.weight_push == "peer":
                self.pusher = PeerWeightPusher(cfg.model, TrainerLayout(tp=cfg.trainer_tp), rtp, self.ps.tp.rank, mine,
                                               self.tag, device, dtype, mtp=cfg.speculative)
        if cfg.weight_push == "broadcast" and (self.is_rollout or (self.is_trainer and self.ps.dp.rank == 0)):
            # one group per source rank of replica 0: a trainer rank takes part in its own group only
            self.bcast = [BroadcastPusher(cfg.model, TrainerLayout(tp=cfg.trainer_tp), rtp, tr[:cfg.trainer_tp], self.engines,
                                          g, device, dtype, src_index=i, mtp=cfg.speculative)
                          for i, g in enumerate(self.bcast_groups) if self.is_rollout or self.rank == tr[i]]
        self.metrics: list = []
        self.stats = {"idle_s": 0.0, "busy_s": 0.0, "sync_ms": [], "push_kernel_ms": [], "rollout_started": []}
        # the engines start from the trainer's initial weights (version 0)
        if self.is_trainer:
            self._push_weights(0)
        else:
            self._wait_for_version(0)

    # ------------------------------------------------------------------ helpers
    def _engine_agree_max(self, value: int) -> int:
        g = self.engine.tp
        if g.size == 1:
            return value
        t = torch.tensor([value], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=g.group)
        return int(t[0])

    # ------------------------------------------------------------------ weight hand-off
    def _n_pushers(self) -> int:
        return len(self.cfg.trainer_ranks)

    def _push_weights(self, version: int) -> float:
        """Trainer side; every trainer rank calls it with the same version."""
        cfg, t0 = self.cfg, time.perf_counter()
        if self.rank == cfg.trainer_ranks[0]:
            self.store.add("wsync/request", version + 1 - self.store.add("wsync/request", 0))   # request = version + 1
        params = dict(self.actor.named_local_params())
        kernel_ms = 0.0
        if cfg.weight_push == "peer":
            self.store.wait_ge(f"wsync/ready/{version}", len(cfg.rollout_ranks), cfg.handshake_timeout_s, cfg.poll_interval,
                               "rollout ranks did not reach a safe point")
            kernel_ms = self.pusher.push(params)
            self.store.add(f"wsync/done/{version}", 1)
        elif self.bcast is not None:
            for b in self.bcast:
                b.sync(params, None)
        ms = (time.perf_counter() - t0) * 1e3
        self.stats["sync_ms"].append(ms)
        self.stats["push_kernel_ms"].append(kernel_ms)
        return ms

    def _maybe_sync_weights(self) -> bool:
        """Rollout side, called at safe points.  Returns True when new weights were taken."""
        req = self.store.add("wsync/request", 0) - 1 if self.is_leader else -1
        req = self._engine_agree_max(req)
        if req <= self.applied_version:
            return False
        self._take_version(req)
        return True

    def _wait_for_version(self, version: int):
        deadline = time.monotonic() + self.cfg.handshake_timeout_s
        while not self._maybe_sync_weights():
            if self.applied_version >= version:
                return
            if time.monotonic() > deadline:
                raise TimeoutError(f"no weights of version {version} arrived within {self.cfg.handshake_timeout_s:.0f} s")
            time.sleep(self.cfg.poll_interval)

    def _take_version(self, version: int):
        cfg = self.cfg
        if self.device.type == "cuda":
            torch.cuda.synchronize()          # nothing that reads the weights is in flight
        self.engine.pause_generation()
        if cfg.weight_push == "peer":
            self.store.add(f"wsync/ready/{version}", 1)
            self.store.wait_ge(f"wsync/done/{version}", self._n_pushers(), cfg.handshake_timeout_s, cfg.poll_interval,
                               "the trainer did not finish its weight push")
        else:
            for b in self.bcast:
                b.sync(None, self.engine.weights)
        if not self.engine.running:
            self.engine.flush_cache()         # cached prefixes were computed with the old weights
        self.engine.update_weight_version(version)
        self.engine.continue_generation()
        self.applied_version = version

    # ------------------------------------------------------------------ rollout pool
    def _generate(self, rid: int) -> list:
        cfg = self.cfg
        per = cfg.rollout_batch_size // len(self.engines)
        groups = self.data_source.get_samples(per * len(self.engines))
        mine = groups[self.engine_id * per:(self.engine_id + 1) * per]
        flat = [s for g in mine for s in g]
        sp = SamplingParams(temperature=cfg.temperature, top_p=cfg.top_p, top_k=cfg.top_k, max_new_tokens=cfg.max_response_len)
        ids = []
        for s_ in flat:
            im = s_.multimodal_train_inputs
            ids.append(self.engine.add_request(s_.tokens, sp, s_.group_index,
                                               **({k: im.get(k) for k in ("pixel_patches", "grid_thw")} if im else {})))
        res = {}
        by_rid = dict(zip(ids, flat))
        parts = max(1, cfg.num_iters_per_train_update)
        chunk = max(1, len(mine) // parts) if parts > 1 else 0      # prompt groups per published part (0: publish at the end)
        left = {id(g): len(g) for g in mine}
        group_of = {id(s_): g for g in mine for s_ in g}
        ready, published = [], 0

        def fill(s, r):
            s.tokens = list(r.prompt) + list(r.output)
            s.response_length = len(r.output)
            s.rollout_log_probs = list(r.logprobs)
            s.weight_versions = sorted(set(r.weight_versions))
            s.status = SampleStatus.TRUNCATED if r.finish_reason == "length" else SampleStatus.COMPLETED
            s.reward = self.reward_fn(s)

        while self.engine.has_work:
            for r in self.engine.step():
                res[r.rid] = r
                if chunk:
                    s_ = by_rid[r.rid]
                    fill(s_, r)
                    g = group_of[id(s_)]
                    left[id(g)] -= 1
                    if left[id(g)] == 0:
                        ready.append(g)
            while chunk and len(ready) >= chunk and published < parts - 1:       # the last part goes out with the seal
                self._publish(rid, [s_ for g in ready[:chunk] for s_ in g], last=False)
                ready, published = ready[chunk:], published + 1
            self._maybe_sync_weights()        # between decode windows
        if chunk:
            return [s_ for g in ready for s_ in g]
        for s, i in zip(flat, ids):
            fill(s, res[i])
        return flat

    def _publish(self, rid: int, samples: list, last: bool):
        """Leader of an engine: advantages per prompt group, rows into the rollout's partition; the engine that
        publishes the last part of all seals it."""
        if not self.is_leader:
            return
        cfg = self.cfg
        part = tq.partition_name(rid)
        if samples:
            batch = convert_samples_to_train_data(
                samples, advantage_estimator=cfg.train.advantage_estimator,
                n_samples_per_prompt=cfg.train.n_samples_per_prompt,
                rewards_normalization=cfg.train.rewards_normalization,
                grpo_std_normalization=cfg.train.grpo_std_normalization)
            self.store.set(f"fields/{rid}", json.dumps(sorted(batch.keys())))
            self.tq.put(batch, part, custom_meta=custom_meta_rows(batch))
        if last and self.store.add(f"puts/{rid}", 1) == len(self.engines):
            self.tq.seal(part)

    def _rollout_loop(self):
        cfg = self.cfg
        for rid in range(cfg.num_rollout):
            deadline = time.monotonic() + cfg.handshake_timeout_s
            while True:
                self._maybe_sync_weights()
                ok = int(satisfy_staleness(self.tq.get_partition_list(), rid - 1, cfg.max_staleness)) if self.is_leader else 1
                if -self._engine_agree_max(-ok):          # minimum over the engine's ranks
                    break
                if time.monotonic() > deadline:
                    raise TimeoutError(f"rollout {rid} waited {cfg.handshake_timeout_s:.0f} s at the staleness gate")
                time.sleep(cfg.poll_interval)
            self.stats["rollout_started"].append((rid, self.applied_version))
            samples = self._generate(rid)
            self._publish(rid, samples, last=True)
        # keep answering weight pushes until the trainer has finished
        deadline = time.monotonic() + cfg.handshake_timeout_s
        while True:
            self._maybe_sync_weights()
            done = self.store.add("trainer_done", 0) if self.is_leader else 0
            if self._engine_agree_max(done):
                break
            if time.monotonic() > deadline:
                raise TimeoutError("the trainer did not finish")
            time.sleep(cfg.poll_interval)
        return self.stats

    # ------------------------------------------------------------------ trainer pool
    FIELDS = ("tokens", "response_lengths", "rewards", "loss_masks", "total_lengths")

    def _fetch(self, rid: int) -> dict:
        """The fetcher waits for the sealed partition and every trainer rank receives all rows."""
        cfg = self.cfg
        box = [None]
        if self.is_fetcher:
            part = tq.partition_name(rid)
            deadline = time.monotonic() + cfg.handshake_timeout_s
            while True:
                if part in self.tq.get_partition_list() and self.tq.check_production_status(list(self.FIELDS), part):
                    fields = json.loads(self.store.get(f"fields/{rid}"))
                    meta = self.tq.get_meta(fields, None, part, "actor", timeout=0.05)
                    if meta is not None:
                        break
                if time.monotonic() > deadline:
                    raise TimeoutError(f"no rollout batch {rid} within {cfg.handshake_timeout_s:.0f} s")
                time.sleep(cfg.poll_interval)
            data = self.tq.get_data(meta)
            box[0] = {k: (v.tolist() if torch.is_tensor(v) else v) for k, v in data.items()}
        if len(cfg.trainer_ranks) > 1:
            dist.broadcast_object_list(box, src=cfg.trainer_ranks[0], group=self.ps.world.group)
        return box[0]

    def _fetch_part(self, rid: int, rows: int):
        """Up to ``rows`` rows of rollout ``rid`` that the trainer has not taken yet - exactly ``rows`` while the engines
        still publish, the remainder once the partition is sealed.  Every trainer rank receives them, with a flag that
        says whether the partition is now used up."""
        cfg = self.cfg
        box = [None]
        if self.is_fetcher:
            part = tq.partition_name(rid)
            deadline = time.monotonic() + cfg.handshake_timeout_s
            meta = None
            while meta is None:
                if part in self.tq.get_partition_list():
                    fields = json.loads(self.store.get(f"fields/{rid}"))
                    meta = self.tq.get_meta(fields, rows, part, "actor", timeout=0.05, allow_partial=True)
                if meta is None:
                    if time.monotonic() > deadline:
                        raise TimeoutError(f"no rows of rollout batch {rid} within {cfg.handshake_timeout_s:.0f} s")
                    time.sleep(cfg.poll_interval)
            data = self.tq.get_data(meta)
            box[0] = ({k: (v.tolist() if torch.is_tensor(v) else v) for k, v in data.items()},
                      bool(self.tq.check_consumption_status("actor", part)))
        if len(cfg.trainer_ranks) > 1:
            dist.broadcast_object_list(box, src=cfg.trainer_ranks[0], group=self.ps.world.group)
        return box[0]

    def _fetch_streamed(self, rid: int):
        """The rollout batch in about ``num_iters_per_train_update`` parts; the forward-only passes (reference and
        old-policy log-probs) run on each part while the engines still generate the rest.  Returns (all rows, this
        replica's forwarded share, seconds spent waiting)."""
        from ..train.actor import concat_batches

        cfg = self.cfg
        unit = cfg.train.n_samples_per_prompt * self.ps.dp.size          # whole prompt groups, equal shares per replica
        rows = cfg.rollout_batch_size * cfg.train.n_samples_per_prompt // cfg.num_iters_per_train_update
        rows = max(unit, rows - rows % unit)
        whole, mine, idle, done = [], [], 0.0, False
        while not done:
            t0 = time.perf_counter()
            data, done = self._fetch_part(rid, rows)
            idle += time.perf_counter() - t0
            whole.append(data)
            mine.append(self.actor.forward_log_probs(self.actor.split_for_dp(dict(data))))
            self.stats["parts_forwarded"] = self.stats.get("parts_forwarded", 0) + 1
        return concat_batches(whole), concat_batches(mine), idle

    def _trainer_loop(self):
        cfg = self.cfg
        t_start = time.perf_counter()
        for rid in range(cfg.num_rollout):
            t0 = time.perf_counter()
            if cfg.num_iters_per_train_update > 1:
                data, batch, idle = self._fetch_streamed(rid)
                self.stats["idle_s"] += idle
                t1 = t0 + idle            # the forward passes count as busy time
            else:
                data = self._fetch(rid)
                self.stats["idle_s"] += time.perf_counter() - t0
                t1 = time.perf_counter()
                batch = self.actor.split_for_dp(data)
            m = self.actor.train(rid, batch)
            self.actor.after_train()
            if self.is_fetcher:
                self.tq.clear_partition(tq.partition_name(rid))
            m["response_tokens"] = float(sum(data["response_lengths"]))
            self.stats["busy_s"] += time.perf_counter() - t1
            if (rid + 1) % cfg.update_weights_interval == 0:
                m["weight_sync_ms"] = self._push_weights(self.actor.weight_version)
                m["weight_push_kernel_ms"] = self.stats["push_kernel_ms"][-1]
            self.metrics.append((rid, m))
        wall = time.perf_counter() - t_start
        if self.rank == cfg.trainer_ranks[0]:
            self.store.add("trainer_done", 1)
        resp = sum(m["response_tokens"] for _, m in self.metrics)
        self.stats.update(wall_s=wall, tokens_per_s=resp / max(wall, 1e-9),
                          trainer_idle_fraction=self.stats["idle_s"] / max(wall, 1e-9))
        return self.metrics

    # ------------------------------------------------------------------ entry points
    def run(self):
        return self._trainer_loop() if self.is_trainer else self._rollout_loop()

    def close(self):
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        if self.engine is not None:
            self.engine.close()
        if self.pusher is not None:
            self.pusher.close()
        dist.barrier()            # importers have unmapped before owners free
        if self.region is not None:
            self.region.close()
        if self.actor is not None and getattr(self.actor, "optimizer", None) is not None:
            self.actor.optimizer.close()
        if self.tq is not None:
            self.tq.close()
        if self.tq_server is not None:
            self.tq_server.close()
        if self.is_rollout and getattr(self, "_shm", None):
            try:
                os.unlink(self._shm)
            except FileNotFoundError:
                pass
