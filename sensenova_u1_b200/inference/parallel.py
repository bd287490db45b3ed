"""Process groups of multi-GPU image sampling.

Ranks are laid out as (guidance branch, token slice): with ``branches`` = 2 (text-to-image with CFG) 2 ranks
sample guidance-parallel, 4 / 8 ranks additionally split every image's tokens over 2 / 4 ranks per branch.
All exchanges go through peer memory from this package's kernels (``inference/engine.py``); the reference has no
multi-GPU sampler of its own (docs/inference_infra.md:20-21 names an external engine for CFG / SP / TP).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class SamplingGroups:
    world: int = 1
    rank: int = 0
    sp: int = 1                    # token slices per guidance branch
    cfg_group: Optional[object] = None
    sp_group: Optional[object] = None
    par_group: Optional[object] = None

    def describe(self) -> str:
        if self.world == 1:
            return "single"
        return f"guidance-parallel x{self.world // self.sp}" + (f" x sequence-parallel x{self.sp}" if self.sp > 1 else "")


def layout(world: int, rank: int, branches: int = 2):
    """(branch, slice, ranks of my slice group, ranks of my branch group) for ``world`` ranks."""
    if world % branches:
        raise ValueError(f"{world} ranks cannot be split over {branches} guidance branches")
    sp = world // branches
    b, s = divmod(rank, sp)
    return b, s, list(range(b * sp, (b + 1) * sp)), [k * sp + s for k in range(branches)]


def init_sampling_groups(branches: int = 2, device: Optional[torch.device] = None) -> SamplingGroups:
    """Reads the torchrun environment, initialises NCCL and creates the groups (every rank creates every group,
    as ``torch.distributed.new_group`` requires)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1:
        return SamplingGroups()
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=device)
    sp = world // branches
    layout(world, rank, branches)                      # validates
    if sp == 1:
        return SamplingGroups(world, rank, 1, dist.group.WORLD, None, None)
    sp_groups = [dist.new_group(list(range(b * sp, (b + 1) * sp))) for b in range(branches)]
    cfg_groups = [dist.new_group([k * sp + s for k in range(branches)]) for s in range(sp)]
    return SamplingGroups(world, rank, sp, cfg_groups[rank % sp], sp_groups[rank // sp], dist.group.WORLD)


def apply_to_model(model, groups: SamplingGroups) -> None:
    """Configures a ``NEOChatModel`` for the groups (no-op on one rank)."""
    if groups.world == 1:
        return
    model.cfg_group = groups.cfg_group
    if groups.sp_group is not None:
        model.enable_sequence_parallel(groups.sp_group, groups.par_group)
