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
        gw, gr = dist.get_world_size(group), dist.get_rank(group)
        base = [int(p) for p in self.handle.buffer_ptrs]
        if self.handle.world_size == gw and self.handle.rank == gr:
            pass
        elif self.handle.world_size == dist.get_world_size() and self.handle.rank == dist.get_rank():
            # the exchange ran over every rank although ``group`` is a sub-group: keep the members' pointers only,
            # in group order, so that stores "to every peer" stay inside the group
            base = [base[g] for g in dist.get_process_group_ranks(group)]
        else:
            raise RuntimeError(f"symmetric memory handle spans {self.handle.world_size} ranks (rank "
                               f"{self.handle.rank}), the group has {gw} (rank {gr})")
        self.world, self.rank = gw, gr
        # the tensor may sit at an offset inside the rendezvoused block
        off = self.tensor.data_ptr() - base[self.rank]
        self.ptrs: List[int] = [b + off for b in base]
        self.c_ptrs = (ctypes.c_longlong * self.world)(*self.ptrs)
        assert self.ptrs[self.rank] == self.tensor.data_ptr()

    def barrier(self):
        self.handle.barrier()


class FlagBarrier:
    """Device-side barrier over a group: one flag word per peer in symmetric memory, a 32-thread
    signal kernel and a 32-thread bounded wait kernel on the calling stream.  After ``barrier()``
    returns control to the stream, everything the peers enqueued before their matching call is
    complete and visible.  On expiry of the wait the device status word carries the error."""

    def __init__(self, group, device):
        self.flags = SymmetricBuffer(dist.get_world_size(group) if group is not None else dist.get_world_size(),
                                     torch.int32, device, group)
        self.world, self.rank = self.flags.world, self.flags.rank
        self.seq = 0
        self.flags.barrier()

    def barrier(self) -> None:
        from ..ops import _lib
        from ..ops._lib import c_int, c_void_p
        self.seq += 1
        st = c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.call("signal_peers", self.flags.c_ptrs, c_int(self.world), c_int(self.rank), c_int(0), c_int(self.seq), st)
        _lib.call("wait_flags", c_void_p(self.flags.tensor.data_ptr()), c_int(self.world), c_int(0), c_int(self.seq), st)


def peer_put(src: torch.Tensor, dst: "SymmetricBuffer", dst_offset_elems: int, skip_self: bool = False) -> None:
    """Copies ``src`` (contiguous) to element offset ``dst_offset_elems`` of ``dst`` on every rank."""
    from ..ops import _lib
    from ..ops._lib import c_int, c_ll, c_void_p
    esz = dst.tensor.element_size()
    assert src.is_contiguous() and src.element_size() == esz
    _lib.call("peer_put", c_void_p(src.data_ptr()), dst.c_ptrs, c_int(dst.world), c_int(dst.rank),
              c_ll(dst_offset_elems * esz), c_ll(src.numel() * esz), c_int(1 if skip_self else 0),
              c_void_p(torch.cuda.current_stream().cuda_stream))


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
