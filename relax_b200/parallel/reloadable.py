"""Process groups that can be torn down and rebuilt.

In colocated mode the trainer's NCCL communicators hold device memory (buffers, channels) that the
rollout engine could use while the trainer sleeps.  The reference monkey-patches ``dist.new_group``
and every collective so communicators are destroyed on ``sleep`` and lazily recreated on
``wake_up`` (relax/utils/reloadable_process_group.py:87-119).  Here a group is an explicit handle:
``ReloadableGroup.group`` creates the communicator on first use; ``destroy_all()`` /
``reload_all()`` act on every live handle.  Creation is collective, so all ranks of the WORLD
must touch a handle in the same order - the registry keeps creation order for ``reload_all``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch.distributed as dist

_HANDLES: List["ReloadableGroup"] = []


class ReloadableGroup:
    def __init__(self, ranks: Sequence[int], backend: Optional[str] = None, timeout=None):
        self.ranks, self.backend, self.timeout = list(ranks), backend, timeout
        self._pg = None
        self.generation = 0
        _HANDLES.append(self)

    @property
    def group(self):
        if self._pg is None:
            kw = {}
            if self.backend:
                kw["backend"] = self.backend
            if self.timeout is not None:
                kw["timeout"] = self.timeout
            self._pg = dist.new_group(self.ranks, **kw)
            self.generation += 1
        return self._pg

    @property
    def alive(self) -> bool:
        return self._pg is not None

    def destroy(self):
        if self._pg is not None:
            if dist.get_rank() in self.ranks:
                dist.destroy_process_group(self._pg)
            self._pg = None


def destroy_all():
    """Free every communicator created through a handle (call on ``sleep``)."""
    for h in _HANDLES:
        h.destroy()


def reload_all():
    """Recreate, in creation order, the communicators of all handles (call on ``wake_up``)."""
    for h in _HANDLES:
        _ = h.group


def forget_all():
    destroy_all()
    _HANDLES.clear()
