"""Pausable device buffers for colocated training and rollout.

``PausableBuffer`` owns device memory whose VIRTUAL address is stable: ``pause()`` gives the physical
memory back to the driver (the trainer can use it), ``resume()`` maps fresh zero-filled memory at the
same address, so CUDA graphs and address tables that reference tensors carved out of the buffer stay
valid across the trainer's turn.  The reference obtains the same effect with the torch_memory_saver
``LD_PRELOAD`` hook around whole allocator regions (relax/distributed/ray/actor_group.py:71-86,
relax/backends/megatron/weight_update/train_offload.py:114-132); this one is explicit and per buffer
(csrc/vmm.cpp).  On CPU (tests) the buffer is an ordinary tensor whose storage is dropped and re-made.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

_DT_SIZE = {torch.bfloat16: 2, torch.float16: 2, torch.float32: 4, torch.int32: 4, torch.int64: 8, torch.uint8: 1}


class PausableBuffer:
    def __init__(self, nbytes: int, device):
        self.device = torch.device(device)
        self.nbytes = int(nbytes)
        self._paused = False
        if self.device.type == "cuda":
            from ..ops import cuda as C

            self._C = C._load()
            self._idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
            self._ptr = self._C.vmm_alloc(self.nbytes, self._idx)
        else:
            self._C, self._ptr = None, 0
            self._cpu = torch.zeros(self.nbytes, dtype=torch.uint8)

    def tensor(self, shape: Sequence[int], dtype: torch.dtype, offset_bytes: int = 0) -> torch.Tensor:
        n = math.prod(shape) * _DT_SIZE[dtype]
        if offset_bytes + n > self.nbytes:
            raise ValueError("view exceeds the buffer")
        if self._C is not None:
            return self._C.tensor_from_ptr(self._ptr + offset_bytes, list(shape), dtype, self._idx)
        return self._cpu[offset_bytes:offset_bytes + n].view(dtype).view(*shape)

    @property
    def paused(self) -> bool:
        return self._paused

    def pause(self):
        """Release the physical memory.  No kernel may touch views of this buffer until :meth:`resume`."""
        if self._paused:
            return
        if self._C is not None:
            self._C.vmm_pause(self._ptr)
        else:
            self._cpu.untyped_storage().resize_(0)
        self._paused = True

    def resume(self):
        if not self._paused:
            return
        if self._C is not None:
            self._C.vmm_resume(self._ptr)
        else:
            self._cpu.untyped_storage().resize_(self.nbytes)
            self._cpu.zero_()
        self._paused = False

    def free(self):
        if self._C is not None and self._ptr:
            self._C.vmm_free(self._ptr)
            self._ptr = 0
