"""Process-group layout of one role (trainer or rollout) inside the job.

One process per GPU.  A *role* owns a contiguous list of global ranks; inside
it ranks are ordered ``tp - cp - ep - dp - pp`` (tp fastest), the same order
the reference asks Megatron for (relax/backends/megatron/initialize.py:37-61).
Groups are ordinary ``torch.distributed`` groups (NCCL on GPUs, gloo on CPU);
the fused kernels additionally use the symmetric heap of
:mod:`relax_b200.parallel.symm_mem` keyed by the same rank lists.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
import torch.distributed as dist


@dataclass
class ParallelDims:
    tp: int = 1
    cp: int = 1
    ep: int = 1
    pp: int = 1
    dp: int = 1

    @property
    def world(self) -> int:
        return self.tp * self.cp * self.dp * self.pp

    def describe(self) -> str:
        parts = [f"{k}{v}" for k, v in (("tp", self.tp), ("cp", self.cp), ("ep", self.ep), ("pp", self.pp), ("dp", self.dp)) if v > 1]
        return "x".join(parts) or "single"


class _Single:
    """Stand-in 'group' for a size-1 dimension (no communicator is created)."""

    size = 1
    rank = 0
    ranks = (0,)
    group = None


@dataclass
class GroupInfo:
    group: Optional[dist.ProcessGroup]
    ranks: tuple
    rank: int  # rank inside the group

    @property
    def size(self) -> int:
        return len(self.ranks)

    @property
    def src(self) -> int:
        return self.ranks[0]


@dataclass
class ParallelState:
    dims: ParallelDims
    global_rank: int
    role_ranks: tuple
    tp: GroupInfo
    cp: GroupInfo
    dp: GroupInfo
    pp: GroupInfo
    ep: GroupInfo
    dp_cp: GroupInfo
    tp_cp: GroupInfo
    world: GroupInfo
    gloo: Optional[dist.ProcessGroup] = None

    # convenient predicates ---------------------------------------------------
    @property
    def is_pp_first(self) -> bool:
        return self.pp.rank == 0

    @property
    def is_pp_last(self) -> bool:
        return self.pp.rank == self.pp.size - 1

    @property
    def is_main(self) -> bool:
        return self.tp.rank == 0 and self.cp.rank == 0 and self.is_pp_last and self.dp.rank == 0

    @property
    def is_data_fetcher(self) -> bool:
        """The rank of each data-parallel replica that talks to the data plane."""
        return self.tp.rank == 0 and self.cp.rank == 0 and self.pp.rank == 0


def _coords(local: int, d: ParallelDims):
    tp_r = local % d.tp
    cp_r = (local // d.tp) % d.cp
    dp_r = (local // (d.tp * d.cp)) % d.dp
    pp_r = local // (d.tp * d.cp * d.dp)
    return tp_r, cp_r, dp_r, pp_r


def _local(tp_r, cp_r, dp_r, pp_r, d: ParallelDims):
    return tp_r + d.tp * (cp_r + d.cp * (dp_r + d.dp * pp_r))


def enumerate_groups(d: ParallelDims):
    """All rank lists (role-local indices) per dimension; pure function so the
    layout can be unit-tested without initialising a process group."""
    out = {k: [] for k in ("tp", "cp", "dp", "pp", "ep", "dp_cp", "tp_cp")}
    for pp_r in range(d.pp):
        for dp_r in range(d.dp):
            for cp_r in range(d.cp):
                out["tp"].append([_local(t, cp_r, dp_r, pp_r, d) for t in range(d.tp)])
            out["tp_cp"].append([_local(t, c, dp_r, pp_r, d) for c in range(d.cp) for t in range(d.tp)])
        for cp_r in range(d.cp):
            for tp_r in range(d.tp):
                out["dp"].append([_local(tp_r, cp_r, x, pp_r, d) for x in range(d.dp)])
        for dp_r in range(d.dp):
            for tp_r in range(d.tp):
                out["cp"].append([_local(tp_r, c, dp_r, pp_r, d) for c in range(d.cp)])
        for tp_r in range(d.tp):
            out["dp_cp"].append([_local(tp_r, c, x, pp_r, d) for x in range(d.dp) for c in range(d.cp)])
            # expert parallel groups are consecutive blocks of the dp x cp ranks
            flat = out["dp_cp"][-1]
            for s in range(0, len(flat), d.ep):
                out["ep"].append(flat[s : s + d.ep])
    for dp_r in range(d.dp):
        for cp_r in range(d.cp):
            for tp_r in range(d.tp):
                out["pp"].append([_local(tp_r, cp_r, dp_r, p, d) for p in range(d.pp)])
    return out


def init_parallel_state(dims: ParallelDims, role_ranks: Optional[Sequence[int]] = None,
                        backend: Optional[str] = None, with_gloo: bool = False) -> ParallelState:
    """Create every group of a role.  Must be called by ALL ranks of the default
    process group (group creation is collective), including ranks outside the role,
    which get ``None`` back."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    me = dist.get_rank() if dist.is_initialized() else 0
    role_ranks = tuple(role_ranks) if role_ranks is not None else tuple(range(world))
    if dims.world != len(role_ranks):
        raise ValueError(f"parallel dims {dims} need {dims.world} ranks, role has {len(role_ranks)}")
    if (dims.dp * dims.cp) % dims.ep:
        raise ValueError("expert-parallel size must divide dp*cp")
    table = enumerate_groups(dims)
    mine: dict[str, GroupInfo] = {}
    for name, lists in table.items():
        for l in lists:
            g_ranks = tuple(role_ranks[i] for i in l)
            grp = None
            if len(g_ranks) > 1 and dist.is_initialized():
                grp = dist.new_group(list(g_ranks), backend=backend)
            if me in g_ranks:
                mine[name] = GroupInfo(grp, g_ranks, g_ranks.index(me))
    wgrp = None
    if dist.is_initialized() and len(role_ranks) > 1:
        wgrp = dist.new_group(list(role_ranks), backend=backend)
    gloo = None
    if with_gloo and dist.is_initialized() and len(role_ranks) > 1:
        gloo = dist.new_group(list(role_ranks), backend="gloo")
    if me not in role_ranks:
        return None
    return ParallelState(
        dims=dims, global_rank=me, role_ranks=role_ranks,
        tp=mine["tp"], cp=mine["cp"], dp=mine["dp"], pp=mine["pp"], ep=mine["ep"],
        dp_cp=mine["dp_cp"], tp_cp=mine["tp_cp"],
        world=GroupInfo(wgrp, role_ranks, role_ranks.index(me)), gloo=gloo,
    )


def single_process_state() -> ParallelState:
    g = GroupInfo(None, (0,), 0)
    return ParallelState(ParallelDims(), 0, (0,), g, g, g, g, g, g, g, g)


def shutdown_distributed(timeout_s: float = 120.0):
    """Leave the process groups in a fixed order that is the same on every rank.

    Two things must have been released by their owners before this is called.  (1) CUDA graphs that captured NCCL
    operations (the rollout engine's decode graphs under tensor parallelism): NCCL's communicator destroy polls
    until every graph referencing the communicator is gone, so with such a graph alive the teardown never returns -
    this is what blocked multi-rank runs of the benchmark (``RolloutEngine.close`` destroys the graphs).
    (2) Symmetric (CUDA IPC) buffers: freeing an exported allocation that a peer still maps is undefined.
    All ranks synchronise their devices and meet; the sub-groups are then
    destroyed one by one, newest first, and the default group last, on the calling thread with its device
    current.  A watchdog thread only observes: if the teardown has not finished after ``timeout_s`` it prints
    which group was being destroyed and ends the process with exit code 3, so a stuck teardown is reported rather
    than hidden.  Returns True when every group was destroyed."""
    import os
    import sys
    import threading

    if not dist.is_initialized():
        return True
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dist.barrier()
    progress = {"at": "start"}
    done = threading.Event()

    def watchdog():
        if not done.wait(timeout_s):
            sys.stderr.write(f"[relax_b200] process-group teardown still running after {timeout_s:.0f} s "
                             f"(rank {os.environ.get('RANK', '0')}, at: {progress['at']}); exiting with code 3\n")
            sys.stderr.flush()
            sys.stdout.flush()
            os._exit(3)

    threading.Thread(target=watchdog, daemon=True).start()
    from torch.distributed import distributed_c10d as c10d

    world = c10d._get_default_group()
    names = dict(c10d._world.pg_names)
    # creation order is the numeric order of the generated names; every rank created every group in the same order
    def order(pg):
        n = names.get(pg, "0")
        return int(n) if str(n).isdigit() else 1 << 30

    subs = sorted((pg for pg in names if pg is not world), key=order, reverse=True)
    for pg in subs:
        progress["at"] = f"sub-group {names.get(pg)}"
        dist.destroy_process_group(pg)
    progress["at"] = "default group"
    dist.destroy_process_group()
    done.set()
    return True
