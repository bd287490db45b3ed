"""Context-parallel attention: one packed sequence split over the ranks of a group.

Every rank holds the query / key / value rows of its own slice of the sequence.  Keys and values
are written into symmetric memory; rank r then walks the W key blocks (its own first, then the
peers' in ring order), pulls a block into local memory with this package's copy kernel (plain peer
loads), runs the packed attention kernel of ``ops/attention.py`` on (local queries x that block)
and folds the partial result into a running (output, log-sum-exp) pair with the ``ring_merge``
kernel.  Masks need no special casing: they derive from per-token metadata (document, position,
image, flags), so any assignment of rows to ranks works, including the zigzag one that balances
causal work (``zigzag_rows``).  Fully masked (query tile, key tile) pairs are skipped by the
kernel's own tile classification, which is what sliding-window / block-causal ring variants
special-case by hand.

Backward: the same walk with the attention backward kernel, given the FINAL log-sum-exp and output
(so every block yields exact partial gradients); dQ partials are summed locally, dK/dV partials
are written per key block into symmetric memory and reduced by the owner with peer loads.

Reference: zigzag double-ring flash attention over NCCL p2p,
training/sensenovalm/model/ops/ring_flash_attn/zigzag_ring_flash_attn_with_sliding_window.py:26-172
(forward), :174-420 (backward); merge utils.py:20-58.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib, attention
from ..ops._lib import c_int, c_ll, c_void_p
from .symm import FlagBarrier, SymmetricBuffer


def zigzag_rows(S: int, world: int, rank: int, block: int = 128) -> torch.Tensor:
    """Row indices of ``rank`` when a sequence of S rows (S a multiple of 2*world*block) is cut into
    2*world chunks and rank r takes chunks r and 2*world-1-r: equal causal work per rank."""
    n = 2 * world
    if S % (n * block):
        raise ValueError(f"S={S} must be a multiple of {n * block}")
    c = S // n
    a = torch.arange(rank * c, (rank + 1) * c)
    b = torch.arange((n - 1 - rank) * c, (n - rank) * c)
    return torch.cat([a, b])


def ring_merge(o_acc, lse_acc, o_blk, lse_blk, out=None, first=False):
    S, H, _ = o_blk.shape
    _lib.call("ring_merge", c_void_p(o_acc.data_ptr()), c_void_p(lse_acc.data_ptr()), c_void_p(o_blk.data_ptr()),
              c_ll(o_blk.stride(0)), c_void_p(lse_blk.data_ptr()), c_void_p(None if out is None else out.data_ptr()),
              c_ll(0 if out is None else out.stride(0)), c_int(S), c_int(H), c_int(1 if first else 0),
              c_void_p(_lib.stream()))


class ContextParallelAttention:
    def __init__(self, group, device, rows: int, n_q_heads: int, n_kv_heads: int, training: bool = True):
        """``rows``: query/key rows per rank (equal on every rank, a multiple of 128).  Collective."""
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.dev = torch.device(device)
        self.S, self.Hq, self.Hk = rows, n_q_heads, n_kv_heads
        kv = rows * n_kv_heads * 128
        # two K/V sets: a fast rank may already write the next exchange while a slow one still reads this one
        self.kv = [SymmetricBuffer(2 * kv, torch.bfloat16, self.dev, self.group) for _ in range(2)]
        self.part = SymmetricBuffer(2 * self.world * kv, torch.bfloat16, self.dev, self.group) if training else None
        self.bar = FlagBarrier(self.group, self.dev)
        self.round = 0
        # two staging slots for peer blocks: block s + 1 is pulled on a side stream while block s is attended to
        self.stage = [torch.empty(2 * kv, dtype=torch.bfloat16, device=self.dev) for _ in range(2)]
        self.side = torch.cuda.Stream(device=self.dev)
        self._ready = [torch.cuda.Event() for _ in range(2)]     # slot holds its block
        self._free = [torch.cuda.Event() for _ in range(2)]      # the kernels that read the slot are queued before this
        self.o_acc = torch.empty(rows, n_q_heads, 128, dtype=torch.float32, device=self.dev)
        self.o_blk = torch.empty(rows, n_q_heads, 128, dtype=torch.bfloat16, device=self.dev)
        self.lse_blk = torch.empty(n_q_heads, rows, dtype=torch.float32, device=self.dev)
        self.delta = torch.empty(n_q_heads, rows, dtype=torch.float32, device=self.dev)
        self.plans: List = []
        self._scratch = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self._published = False

    # ---- per batch ----------------------------------------------------------------------------
    def set_metadata(self, meta_local: torch.Tensor) -> None:
        """``meta_local`` [rows,4] int32 (``ops.attention.make_meta``) of this rank's rows; gathers the
        metadata of every rank and classifies the tiles of each (local queries, key block) pair."""
        metas = [torch.empty_like(meta_local) for _ in range(self.world)]
        dist.all_gather(metas, meta_local.contiguous(), group=self.group)
        self.plans = [attention.build_plan(meta_local, m) for m in metas]

    # ---- exchange -----------------------------------------------------------------------------
    def kv_views(self):
        """(k, v) [rows, Hk, 128] views of the symmetric buffers of the current round."""
        t = self.kv[self.round & 1].tensor
        n = self.S * self.Hk * 128
        return t[:n].view(self.S, self.Hk, 128), t[n:].view(self.S, self.Hk, 128)

    def publish(self, k, v) -> None:
        """Starts a new exchange round with this rank's keys / values ([rows, Hk, 128], any row
        stride).  The other K/V set is used than in the previous round, so a rank that is ahead
        never overwrites what a slower rank still reads; the barrier that makes the data visible
        is taken by the next ``forward`` / ``backward``."""
        self.round += 1
        kk, vv = self.kv_views()
        kk.copy_(k)
        vv.copy_(v)
        self._published = True

    def _sync_round(self) -> None:
        if self._published:
            self.bar.barrier()                   # every rank's K/V of this round is complete
            self._published = False

    def _start_pulls(self) -> None:
        """After the round's barrier: the side stream may read the peers' K/V from here on, both slots are free."""
        cur = torch.cuda.current_stream()
        for e in self._free:
            e.record(cur)
        self._prefetch(1)

    def _prefetch(self, s: int) -> None:
        """Queues the pull of the block of step ``s`` (rank + s) into slot ``s & 1`` on the side stream."""
        if s >= self.world:
            return
        j = (self.rank + s) % self.world
        n = self.S * self.Hk * 128
        slot = s & 1
        self.side.wait_event(self._free[slot])
        _lib.call("copy_bytes", c_void_p(self.kv[self.round & 1].ptrs[j]), c_void_p(self.stage[slot].data_ptr()),
                  c_ll(2 * n * 2), c_void_p(self.side.cuda_stream))
        self._ready[slot].record(self.side)

    def _block(self, s: int):
        """K/V of step ``s`` (rank + s) for this round in local memory (own block, s = 0: in place); the pull of the
        next step's block is queued first, so that it runs beside this step's attention."""
        n = self.S * self.Hk * 128
        if s == 0:
            t = self.kv[self.round & 1].tensor
        else:
            self._prefetch(s + 1)
            torch.cuda.current_stream().wait_event(self._ready[s & 1])
            t = self.stage[s & 1]
        return t[:n].view(self.S, self.Hk, 128), t[n:].view(self.S, self.Hk, 128)

    def _release(self, s: int) -> None:
        if s > 0:
            self._free[s & 1].record(torch.cuda.current_stream())

    def forward(self, q, scale: float, out=None, lse=None):
        """q [rows,Hq,128]; K/V of this round come from ``publish``.  Returns (out bf16, lse fp32)."""
        if out is None:
            out = torch.empty_like(q)
        if lse is None:
            lse = torch.empty(self.Hq, self.S, dtype=torch.float32, device=self.dev)
        self._sync_round()
        self._start_pulls()
        for s in range(self.world):
            j = (self.rank + s) % self.world
            k, v = self._block(s)
            attention.attention_fwd(q, k, v, self.plans[j], scale, out=self.o_blk, lse=self.lse_blk)
            self._release(s)
            ring_merge(self.o_acc, lse, self.o_blk, self.lse_blk, out=out if s == self.world - 1 else None, first=s == 0)
        return out, lse

    def backward(self, q, o, dout, lse, scale: float, dq=None, dk=None, dv=None):
        """Gradients for the K/V set of the current round."""
        self._sync_round()
        W, n = self.world, self.S * self.Hk * 128
        dq = torch.empty_like(q) if dq is None else dq
        dq_acc = self.o_acc                     # fp32 [rows,Hq,128], free after the forward
        part = self.part.tensor
        self._start_pulls()
        for s in range(W):
            j = (self.rank + s) % W
            k, v = self._block(s)
            dkj = part[(2 * j) * n:(2 * j + 1) * n].view(self.S, self.Hk, 128)
            dvj = part[(2 * j + 1) * n:(2 * j + 2) * n].view(self.S, self.Hk, 128)
            attention.attention_bwd(q, k, v, o, dout, lse, self.plans[j], scale, dq=self.o_blk, dk=dkj, dv=dvj,
                                    delta=self.delta)
            self._release(s)
            if s == 0:
                dq_acc.copy_(self.o_blk)
            else:
                dq_acc.add_(self.o_blk)
        dq.copy_(dq_acc)
        self.bar.barrier()                       # every rank's partial dK/dV blocks are complete
        off = 2 * self.rank * n
        _lib.call("zero_rs_sumsq", self.part.c_ptrs, c_int(W), c_int(self.rank), c_ll(off), c_ll(2 * n),
                  c_void_p(None), c_int(0), c_int(0), c_void_p(self._scratch.data_ptr()), c_void_p(_lib.stream()))
        mine = part[off:off + 2 * n]
        dk = mine[:n].view(self.S, self.Hk, 128) if dk is None else dk.copy_(mine[:n].view(self.S, self.Hk, 128))
        dv = mine[n:].view(self.S, self.Hk, 128) if dv is None else dv.copy_(mine[n:].view(self.S, self.Hk, 128))
        self.bar.barrier()                       # peers are done reading my partials
        return dq, dk, dv
