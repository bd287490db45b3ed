"""Symmetric (peer-mapped) device memory for the kernels that do their own collectives.

Allocation and handle exchange ride on ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations whose handles are exchanged over the process group's store); everything that
moves data is a kernel of this package that dereferences the peer pointers returned here.
No multicast object is requested: the kernels use plain peer loads and stores.
(The reference has no such layer: it only calls NCCL through torch.distributed,
training/sensenovalm/core/parallel/comm/utils.py:35-276.)
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Tuple

import torch
import torch.distributed as dist


class SymmetricBuffer:
    """A tensor that exists at the same size on every rank of ``group`` with all peers mapped."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        group = group if group is not None else dist.group.WORLD
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group=group)
        self.world = self.handle.world_size
        self.rank = self.handle.rank
        esz = self.tensor.element_size()
        base = [int(p) for p in self.handle.buffer_ptrs]
        # the tensor may sit at an offset inside the rendezvoused block
        off = self.tensor.data_ptr() - base[self.rank]
        self.ptrs: List[int] = [b + off for b in base]
        self.c_ptrs = (ctypes.c_longlong * self.world)(*self.ptrs)
        assert self.ptrs[self.rank] == self.tensor.data_ptr()

    def barrier(self):
        self.handle.barrier()


def symmetric_arenas(store, group=None) -> None:
    """Moves the ``mat``/``vec`` weight and gradient arenas of ``store`` into symmetric memory
    (contents are preserved) and records the peer pointer tables on the store."""
    store.symm = {"arena": {}, "grad": {}}
    for kind, arenas in (("arena", store.arena), ("grad", store.grad_arena)):
        for a, t in list(arenas.items()):
            if a == "exp":          # this rank's experts only: no peer reads them
                continue
            sb = SymmetricBuffer(t.numel(), t.dtype, t.device, group)
            sb.tensor.copy_(t)
            arenas[a] = sb.tensor
            store.symm[kind][a] = sb
    store.rebind_views()
