"""Expert parallelism over NVLink peer memory.

Rank r of the expert-parallel group holds experts ``[r * E/ep, (r + 1) * E/ep)`` of every mixture.
Token rows travel to the owning rank and back by peer stores / peer loads issued from this
package's own kernels (csrc/moe.cu: ``moe_ep_*``): there is no all-to-all collective, no split
size ever reaches the host, and the only synchronisation is a flag barrier in symmetric memory
(one 32-thread signal kernel + one 32-thread bounded wait kernel on the compute stream).

The reference does the same job with two ``all_to_all_single`` calls per direction whose split
sizes are synchronised through the host (training/sensenovalm/model/moe/dropless_layer_qwen.py:
407-506 dispatch, 662-773 combine; training/sensenovalm/model/moe/utils.py:15-80).

Per mixture this object owns four receive-side buffers in symmetric memory:

* ``xp``   rows dispatched to this rank's experts (written by every source rank),
* ``yp``   expert outputs (read by the source ranks in ``combine``),
* ``dyp``  gradients of ``yp`` (written by the source ranks in the backward of ``combine``),
* ``dxp``  gradients of ``xp`` (read by the source ranks in the backward of ``dispatch``),

each ``capacity`` rows: ``capacity_factor`` x the mean number of rows per rank, plus one padding
tile per local expert.  ``capacity_factor=None`` sizes them for the worst case (every copy of every
rank lands on one rank: factor = world size), which is what keeps routing dropless under any load;
with a smaller factor a rank that attracts more rows than fit reports an error through the device
status word, and the copies that did not fit are skipped by dispatch and combine (never an
out-of-range access).  Only the rows in use are touched: GEMM tiles, activation kernels and the
clearing of padding rows all stop at the device-side row count.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch
import torch.distributed as dist

from .symm import FlagBarrier, SymmetricBuffer


@dataclass
class EpBuffers:
    xp: SymmetricBuffer
    yp: SymmetricBuffer
    dyp: SymmetricBuffer
    dxp: SymmetricBuffer
    counts_all: SymmetricBuffer
    capacity: int
    H: int

    def view(self, which: str) -> torch.Tensor:
        return getattr(self, which).tensor.view(self.capacity, self.H)


class ExpertParallel:
    def __init__(self, group, device, hidden: int, mixtures: Dict[str, tuple], max_tokens: int,
                 capacity_factor: float | None = 2.0, training: bool = True):
        """``mixtures``: name -> (experts, top-k).  ``max_tokens``: the most rows one rank routes
        through a mixture in one call.  Collective: every rank of ``group`` must construct it."""
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("peer-memory expert parallelism spans one NVLink domain (<= 8 ranks)")
        self.dev = torch.device(device)
        self.bufs: Dict[str, EpBuffers] = {}
        for name, (E, K) in mixtures.items():
            if E % self.world:
                raise ValueError(f"mixture {name}: {E} experts do not split over {self.world} ranks")
            e_loc = E // self.world
            factor = float(self.world) if capacity_factor is None else min(float(capacity_factor), float(self.world))
            cap = (int(max_tokens * K * factor) + 127) // 128 * 128 + e_loc * 128
            mk = lambda: SymmetricBuffer(cap * hidden, torch.bfloat16, self.dev, self.group)
            one = SymmetricBuffer(8, torch.bfloat16, self.dev, self.group) if not training else None
            self.bufs[name] = EpBuffers(mk(), mk(), mk() if training else one, mk() if training else one,
                                        SymmetricBuffer(self.world * E, torch.int32, self.dev, self.group), cap, hidden)
        self._bar = FlagBarrier(self.group, self.dev)

    def barrier(self) -> None:
        """Device-side barrier on the current stream (see ``symm.FlagBarrier``)."""
        self._bar.barrier()
