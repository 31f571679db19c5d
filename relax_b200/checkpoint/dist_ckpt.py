"""Sharded trainer checkpoints in the ``torch.distributed.checkpoint`` on-disk format
with Megatron's directory conventions.

Layout (relax/backends/megatron/model.py:1578-1606, relax/utils/utils.py:613-620):

    <save>/latest_checkpointed_iteration.txt
    <save>/iter_0000012/.metadata            pickled torch.distributed.checkpoint Metadata
    <save>/iter_0000012/__<rank>_0.distcp    this rank's shards (torch.save blobs at recorded offsets)
    <save>/iter_0000012/common.pt            step, config, RNG, data-source cursor

Every model tensor is recorded under its GLOBAL (unsharded) name and shape; a rank
contributes the N-d boxes it owns (TP row/column shards, expert slices, pipeline
layers renumbered globally).  Because the index is a standard DCP ``Metadata`` object,
``torch.distributed.checkpoint.load`` can read these checkpoints, and
:func:`load_full_tensors` reads any DCP checkpoint whose tensors are plain chunked
tensors (the form Megatron's ``torch_dist`` format stores) - so parallel layouts can
change between save and load.  Optimizer state is stored per parameter as flat 1-D
tensors (``optimizer.state.<kind>.<param>``) chunked by the distributed-optimizer shards.
"""
from __future__ import annotations

import io
import os
import pickle
import re
import shutil
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
from torch.distributed.checkpoint.filesystem import _StorageInfo
from torch.distributed.checkpoint.metadata import (BytesStorageMetadata, ChunkStorageMetadata, Metadata, MetadataIndex,
                                                   TensorProperties, TensorStorageMetadata)

from ..models.config import ModelConfig
from ..parallel.state import ParallelState

TRACKER = "latest_checkpointed_iteration.txt"


def iter_dir(save: str, iteration: int) -> str:
    return os.path.join(save, f"iter_{iteration:07d}")


def read_latest_iteration(path: Optional[str]) -> Optional[int]:
    if not path:
        return None
    try:
        return int(open(os.path.join(path, TRACKER)).read().strip())
    except (OSError, ValueError):
        return None


def is_dist_checkpoint(path: str) -> bool:
    it = read_latest_iteration(path)
    return it is not None and os.path.exists(os.path.join(iter_dir(path, it), ".metadata"))


# ----------------------------------------------------------------------------- shard geometry


@dataclass
class Shard:
    fqn: str
    global_shape: tuple
    offsets: tuple
    tensor: torch.Tensor


def shard_of_param(cfg: ModelConfig, ps: ParallelState, name: str, p: torch.Tensor, layer_offset: int = 0) -> Shard:
    """Global name, global shape and offsets of a local parameter."""
    tp, r = ps.tp.size, ps.tp.rank
    m = re.match(r"decoder\.layers\.(\d+)\.(.+)", name)
    gname = name
    if m:
        gname = f"decoder.layers.{int(m.group(1)) + layer_offset}.{m.group(2)}"
    shape, off = list(p.shape), [0] * p.dim()
    col_parallel = ("linear_qkv.weight", "linear_qkv.bias", "word_embeddings.weight", "output_layer.weight")
    if name.endswith(col_parallel):
        shape[0] *= tp
        off[0] = r * p.shape[0]
    elif name.endswith("mlp.linear_fc1.weight"):
        # local = [gate_r ; up_r]: two boxes of the global [gate ; up]; handled by the caller via split_fc1
        shape[0] *= tp
    elif name.endswith(("linear_proj.weight", "mlp.linear_fc2.weight")) and "experts" not in name:
        shape[1] *= tp
        off[1] = r * p.shape[1]
    elif "mlp.experts." in name:
        shape[0] *= ps.ep.size
        off[0] = ps.ep.rank * p.shape[0]
    return Shard(gname, tuple(shape), tuple(off), p)


def local_shards(cfg: ModelConfig, ps: ParallelState, named_params, layer_offset: int = 0) -> list[Shard]:
    out = []
    tp, r = ps.tp.size, ps.tp.rank
    for name, p in named_params:
        p = p.detach()
        s = shard_of_param(cfg, ps, name, p, layer_offset)
        if name.endswith("mlp.linear_fc1.weight") and "experts" not in name and tp > 1:
            fl = p.shape[0] // 2
            F = fl * tp
            out.append(Shard(s.fqn, s.global_shape, (r * fl, 0), p[:fl]))
            out.append(Shard(s.fqn, s.global_shape, (F + r * fl, 0), p[fl:]))
        else:
            out.append(s)
    return out


def owns_replicated(ps: ParallelState, name: str) -> bool:
    """Replicated tensors (norms, router) are written once: by TP rank 0 of DP/CP rank 0."""
    return ps.tp.rank == 0


# ----------------------------------------------------------------------------- save


def save_checkpoint(save: str, iteration: int, cfg: ModelConfig, ps: ParallelState, model, optimizer=None,
                    extra: Optional[dict] = None, layer_offset: int = 0, save_optim: bool = True) -> str:
    """Collective over the role's ranks.  Model tensors are written by the first
    data-parallel replica only; optimizer shards by every rank."""
    d = iter_dir(save, iteration)
    rank = ps.world.rank
    if rank == 0:
        os.makedirs(d, exist_ok=True)
    if ps.world.size > 1:
        dist.barrier(group=ps.world.group)
    fname = f"__{rank}_0.distcp"
    records = []   # (fqn, global_shape, offsets, sizes, dtype, file offset, length)
    with open(os.path.join(d, fname), "wb") as f:
        def write(fqn, gshape, offs, t):
            buf = io.BytesIO()
            torch.save(t.detach().cpu().contiguous().clone(), buf)
            b = buf.getvalue()
            records.append((fqn, tuple(gshape), tuple(offs), tuple(t.shape), t.dtype, f.tell(), len(b)))
            f.write(b)

        if ps.dp_cp.rank == 0:
            replicated = {n for n, p in model.named_parameters() if getattr(p, "tp_replicated", False)}
            for s in local_shards(cfg, ps, model.named_parameters(), layer_offset):
                base = re.sub(r"decoder\.layers\.\d+\.", "", s.fqn)
                is_rep = any(re.sub(r"decoder\.layers\.\d+\.", "", n) == base for n in replicated)
                if is_rep and ps.tp.rank != 0:
                    continue
                if "mlp.experts." not in s.fqn and ps.ep.size > 1 and False:
                    continue
                write(s.fqn, s.global_shape, s.offsets, s.tensor)
        if optimizer is not None and save_optim:
            sd = optimizer.state_dict()
            lo, hi = sd["shard"]
            tag = f"tp{ps.tp.rank}"
            for kind in ("master", "exp_avg", "exp_avg_sq"):
                fq = f"optimizer.state.{kind}.flat.{tag}"
                write(fq, (sd["total"],), (lo,), sd[kind])
    gathered = [None] * ps.world.size
    if ps.world.size > 1:
        dist.all_gather_object(gathered, (fname, records), group=ps.world.group)
    else:
        gathered = [(fname, records)]
    if rank == 0:
        sdm, storage = {}, {}
        for fn, recs in gathered:
            for fqn, gshape, offs, sizes, dtype, foff, ln in recs:
                md = sdm.get(fqn)
                if md is None:
                    md = sdm[fqn] = TensorStorageMetadata(TensorProperties(dtype=dtype), torch.Size(gshape), [])
                md.chunks.append(ChunkStorageMetadata(torch.Size(offs), torch.Size(sizes)))
                storage[MetadataIndex(fqn, torch.Size(offs))] = _StorageInfo(fn, foff, ln)
        meta = Metadata(state_dict_metadata=sdm, storage_data=storage)
        with open(os.path.join(d, ".metadata"), "wb") as f:
            pickle.dump(meta, f)
        common = {"iteration": iteration, "model_config": cfg.to_dict(), "parallel": vars(ps.dims),
                  "optimizer_step": optimizer.step_count if optimizer is not None else 0}
        common.update(extra or {})
        torch.save(common, os.path.join(d, "common.pt"))
        with open(os.path.join(save, TRACKER), "w") as f:
            f.write(str(iteration))
    if ps.world.size > 1:
        dist.barrier(group=ps.world.group)
    return d


# ----------------------------------------------------------------------------- load


def read_metadata(ckpt_dir: str) -> Metadata:
    with open(os.path.join(ckpt_dir, ".metadata"), "rb") as f:
        return pickle.load(f)


def load_box(ckpt_dir: str, meta: Metadata, fqn: str, offsets, sizes) -> torch.Tensor:
    """Read an arbitrary N-d box of a saved tensor by assembling the chunks that intersect it."""
    md = meta.state_dict_metadata[fqn]
    out = torch.empty(tuple(sizes), dtype=md.properties.dtype)
    filled = 0
    for ch in md.chunks:
        lo = [max(o, co) for o, co in zip(offsets, ch.offsets)]
        hi = [min(o + s, co + cs) for o, s, co, cs in zip(offsets, sizes, ch.offsets, ch.sizes)]
        if any(l >= h for l, h in zip(lo, hi)):
            continue
        info = meta.storage_data[MetadataIndex(fqn, ch.offsets)]
        with open(os.path.join(ckpt_dir, info.relative_path), "rb") as f:
            f.seek(info.offset)
            t = torch.load(io.BytesIO(f.read(info.length)), map_location="cpu", weights_only=True)
        src = tuple(slice(l - co, h - co) for l, h, co in zip(lo, hi, ch.offsets))
        dst = tuple(slice(l - o, h - o) for l, h, o in zip(lo, hi, offsets))
        out[dst] = t[src]
        n = 1
        for l, h in zip(lo, hi):
            n *= h - l
        filled += n
    if filled < out.numel():
        raise KeyError(f"{fqn}: box {tuple(offsets)}+{tuple(sizes)} is not fully covered by the checkpoint")
    return out


def load_full_tensors(ckpt_dir: str, names=None) -> dict:
    meta = read_metadata(ckpt_dir)
    out = {}
    for fqn, md in meta.state_dict_metadata.items():
        if isinstance(md, BytesStorageMetadata) or (names is not None and fqn not in names):
            continue
        out[fqn] = load_box(ckpt_dir, meta, fqn, [0] * len(md.size), list(md.size))
    return out


def load_checkpoint(load: str, cfg: ModelConfig, ps: ParallelState, model, optimizer=None, iteration: Optional[int] = None,
                    layer_offset: int = 0, load_optim: bool = True) -> dict:
    """Load into the current parallel layout (which may differ from the saving one).
    Returns the ``common.pt`` dictionary."""
    it = iteration if iteration is not None else read_latest_iteration(load)
    if it is None:
        raise FileNotFoundError(f"no {TRACKER} under {load}")
    d = iter_dir(load, it)
    meta = read_metadata(d)
    with torch.no_grad():
        for s in local_shards(cfg, ps, model.named_parameters(), layer_offset):
            t = load_box(d, meta, s.fqn, s.offsets, s.tensor.shape)
            s.tensor.copy_(t.to(s.tensor.dtype))
    common = torch.load(os.path.join(d, "common.pt"), weights_only=False)
    if optimizer is not None:
        optimizer.reload_master_from_params()
        tag = f"tp{ps.tp.rank}"
        key = f"optimizer.state.master.flat.{tag}"
        same_layout = key in meta.state_dict_metadata and tuple(meta.state_dict_metadata[key].size) == (optimizer.total,)
        if load_optim and same_layout:
            lo, hi = optimizer.lo, optimizer.hi
            sd = {"step": common.get("optimizer_step", 0)}
            for kind in ("master", "exp_avg", "exp_avg_sq"):
                sd[kind] = load_box(d, meta, f"optimizer.state.{kind}.flat.{tag}", [lo], [hi - lo])
            optimizer.load_state_dict(sd)
    return common


# ----------------------------------------------------------------------------- rotation


def rotate_checkpoints(save: str, keep: Optional[int]):
    """Keep the newest ``keep`` ``iter_*`` directories (relax/utils/rotate_ckpt.py:17-79)."""
    if not keep or keep <= 0 or not os.path.isdir(save):
        return []
    its = sorted(int(m.group(1)) for m in (re.fullmatch(r"iter_(\d+)", n) for n in os.listdir(save)) if m)
    removed = []
    for it in its[:-keep]:
        shutil.rmtree(iter_dir(save, it), ignore_errors=True)
        removed.append(it)
    return removed


def resolve_start_rollout_id(load: Optional[str], explicit: Optional[int] = None) -> int:
    """Where training resumes: an explicit ``--start-rollout-id`` wins, else the iteration after the
    latest checkpoint, else 0 (relax/components/actor.py:25-40)."""
    if explicit is not None:
        return explicit
    it = read_latest_iteration(load)
    return 0 if it is None else it + 1


@torch.no_grad()
def load_full_state(cfg: ModelConfig, ps: ParallelState, model, full_state: dict, strict: bool = True) -> list:
    """Copy this rank's boxes out of a FULL (unsharded, Megatron-layout) state dict into the local parameters - the
    path from a Hugging Face checkpoint into any TP / EP / PP layout.  Vocabulary rows past the checkpoint's size
    (padding to a multiple of TP) are zeroed.  Returns the names that were not found (raises when ``strict``)."""
    per = cfg.num_layers // ps.pp.size
    missing = []
    for s in local_shards(cfg, ps, model.named_parameters(), layer_offset=ps.pp.rank * per):
        src = full_state.get(s.fqn)
        if src is None:
            missing.append(s.fqn)
            continue
        idx = tuple(slice(o, o + n) for o, n in zip(s.offsets, s.tensor.shape))
        box = src[idx]
        if box.shape != s.tensor.shape:                      # padded vocabulary shard
            s.tensor.zero_()
            s.tensor[tuple(slice(0, n) for n in box.shape)].copy_(box)
        else:
            s.tensor.copy_(box)
    if missing and strict:
        raise KeyError(f"{len(missing)} parameters missing from the checkpoint, e.g. {missing[:3]}")
    return missing
