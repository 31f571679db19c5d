"""Training profiler: a ``torch.profiler`` window over chosen steps, CUDA memory-history snapshots,
and a per-step record of allocator statistics (relax/utils/profile_utils.py ``TrainProfiler``,
relax/utils/memory_utils.py).  All of it is opt-in and costs nothing when disabled.
"""
from __future__ import annotations

import os
from typing import Optional

import torch


def memory_stats(device=None) -> dict:
    if not torch.cuda.is_available():
        return {}
    free, total = torch.cuda.mem_get_info(device)
    return {
        "mem/allocated_gb": torch.cuda.memory_allocated(device) / 2**30,
        "mem/reserved_gb": torch.cuda.memory_reserved(device) / 2**30,
        "mem/max_allocated_gb": torch.cuda.max_memory_allocated(device) / 2**30,
        "mem/free_gb": free / 2**30,
        "mem/total_gb": total / 2**30,
    }


class TrainProfiler:
    """``step()`` once per training step.  Profiles steps ``[start, end)`` and writes a Chrome trace
    per rank under ``out_dir``; optionally records the CUDA allocator history over the same window."""

    def __init__(self, out_dir: Optional[str], start_step: int = -1, end_step: int = -1, rank: int = 0,
                 with_stack: bool = False, record_memory: bool = False, record_shapes: bool = False):
        self.out_dir, self.start, self.end, self.rank = out_dir, start_step, end_step, rank
        self.with_stack, self.record_memory, self.record_shapes = with_stack, record_memory, record_shapes
        self.enabled = out_dir is not None and 0 <= start_step < end_step
        self._step = 0
        self._prof = None
        self.trace_path = None

    def _begin(self):
        os.makedirs(self.out_dir, exist_ok=True)
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
            if self.record_memory:
                torch.cuda.memory._record_memory_history(max_entries=100000)
        self._prof = torch.profiler.profile(activities=acts, with_stack=self.with_stack, record_shapes=self.record_shapes)
        self._prof.__enter__()

    def _finish(self):
        self._prof.__exit__(None, None, None)
        self.trace_path = os.path.join(self.out_dir, f"trace_rank{self.rank}_steps{self.start}-{self.end}.json")
        self._prof.export_chrome_trace(self.trace_path)
        if self.record_memory and torch.cuda.is_available():
            torch.cuda.memory._dump_snapshot(os.path.join(self.out_dir, f"memory_rank{self.rank}.pickle"))
            torch.cuda.memory._record_memory_history(enabled=None)
        self._prof = None

    def step(self):
        if not self.enabled:
            return
        if self._step == self.start:
            self._begin()
        self._step += 1
        if self._prof is not None and self._step == self.end:
            self._finish()

    def close(self):
        if self._prof is not None:
            self._finish()


class MemorySnapshotter:
    """``--memory-snapshot-dir`` / ``--memory-snapshot-num-steps`` (relax/utils/memory_utils.py): record the CUDA
    caching allocator's history from the first training step and dump one snapshot per rank (the pickle that
    https://pytorch.org/memory_viz reads) after ``num_steps`` steps - independent of the kernel-trace window."""

    def __init__(self, out_dir: Optional[str], num_steps: Optional[int] = None, rank: int = 0, max_entries: int = 200000):
        self.out_dir, self.num_steps, self.rank, self.max_entries = out_dir, int(num_steps or 1), rank, max_entries
        self.enabled = out_dir is not None and torch.cuda.is_available()
        self._step, self.path, self._on = 0, None, False

    def step(self):
        if not self.enabled or self.path is not None:
            return
        if self._step == 0:
            os.makedirs(self.out_dir, exist_ok=True)
            torch.cuda.memory._record_memory_history(max_entries=self.max_entries)
            self._on = True
        self._step += 1
        if self._step > self.num_steps:
            self.dump()

    def dump(self):
        if self._on and self.path is None:
            self.path = os.path.join(self.out_dir, f"memory_snapshot_rank{self.rank}.pickle")
            torch.cuda.memory._dump_snapshot(self.path)
            torch.cuda.memory._record_memory_history(enabled=None)
            self._on = False

    def close(self):
        self.dump()
