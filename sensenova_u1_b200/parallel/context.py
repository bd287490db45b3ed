"""Parallel context: the rank grid and the process groups of every parallel mode.

Same modes and ordering rules as the reference's ``ParallelContext`` / ``ParallelMode``
(training/sensenovalm/core/context/parallel_context.py:521-723,
process_group_initializer.py:23-91, 280-342): the global ranks form a grid whose fastest
axis is tensor (ISP: sequence) parallel, then weight parallel, then data, then pipeline;
``zero1`` groups subdivide the (weight-)data group; expert groups re-tile the data x tensor
plane.  Unlike the reference there is no global singleton: a ``ParallelContext`` object is
passed to whoever needs it, and it works on gloo (CPU tests) and NCCL alike.
"""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


class ParallelMode(enum.Enum):
    GLOBAL = "global"
    DATA = "data"
    TENSOR = "tensor"           # Megatron TP / SP, or Ulysses sequence parallel under ISP
    WEIGHT = "weight"           # ISP weight parallel (ZeRO-3-like)
    WEIGHT_DATA = "weight_data"
    PIPELINE = "pipeline"
    ZERO1 = "zero1"
    EXPERT = "expert"
    EXPERT_DATA = "expert_data"
    EXPERT_WEIGHT = "expert_weight"
    EXPERT_ZERO1 = "expert_zero1"
    COMMON_DATA = "common_data"  # ranks that must see the same batch (tensor x weight plane)


@dataclass
class ParallelConfig:
    tensor: int = 1
    tensor_mode: str = "mtp"     # mtp | msp | fsp | isp
    weight: int = 1
    pipeline: int = 1
    zero1: int = -1              # -1: the whole data-parallel group
    expert: int = 1
    expert_weight: int = 1
    expert_zero1: int = -1

    @classmethod
    def from_dict(cls, d: dict) -> "ParallelConfig":
        """Accepts the reference config schema: values may be ints or dicts with ``size``."""
        def size(v, default=1):
            if v is None:
                return default
            return int(v.get("size", default)) if isinstance(v, dict) else int(v)
        t = d.get("tensor", 1)
        return cls(tensor=size(t), tensor_mode=(t.get("mode", "mtp") if isinstance(t, dict) else "mtp"),
                   weight=size(d.get("weight", 1)), pipeline=size(d.get("pipeline", 1)),
                   zero1=size(d.get("zero1", -1), -1), expert=size(d.get("expert", 1)),
                   expert_weight=size(d.get("expert_weight", 1)), expert_zero1=size(d.get("expert_zero1", -1), -1))


def _check(cond, msg):
    if not cond:
        raise ValueError(msg)


class ParallelContext:
    def __init__(self, cfg: ParallelConfig, rank: Optional[int] = None, world_size: Optional[int] = None,
                 create_groups: bool = True, backend: Optional[str] = None):
        self.cfg = cfg
        self.rank = dist.get_rank() if rank is None else rank
        self.world_size = dist.get_world_size() if world_size is None else world_size
        ws, tp, wp, pp = self.world_size, cfg.tensor, cfg.weight, cfg.pipeline
        _check(ws % (tp * pp) == 0, f"world size {ws} is not a multiple of tensor {tp} x pipeline {pp}")
        _check(wp == 1 or cfg.tensor_mode == "isp", "weight parallel needs tensor mode 'isp'")
        self.dp = ws // (tp * pp)
        _check(self.dp % 1 == 0 and (ws // pp) % (tp * wp) == 0 or wp == 1,
               f"weight parallel {wp} does not divide the stage size {ws // pp}")
        if wp > 1:
            _check((ws // pp // tp) % wp == 0, "weight parallel must divide data x weight plane")
        self.wdp = ws // (tp * pp * wp)              # weight-data parallel size
        zero_base = self.wdp if wp > 1 else self.dp
        self.zero1 = zero_base if cfg.zero1 in (-1, 0) else cfg.zero1
        _check(zero_base % self.zero1 == 0, f"zero1 {self.zero1} must divide {zero_base}")
        ep = cfg.expert
        _check((self.dp * tp) % max(ep, 1) == 0, f"expert parallel {ep} must divide data x tensor {self.dp * tp}")
        self.sizes: Dict[ParallelMode, int] = {}
        self.ranks_in_group: Dict[ParallelMode, List[int]] = {}
        self.groups: Dict[ParallelMode, object] = {}
        self.local_rank: Dict[ParallelMode, int] = {}
        self._build(create_groups, backend)

    # rank = ((pp_idx * dp + dp_idx) * tp + tp_idx), with the data axis split as dp_idx = wdp_idx * wp + wp_idx
    def coords(self, rank: int):
        tp, wp = self.cfg.tensor, self.cfg.weight
        tp_i = rank % tp
        dp_i = (rank // tp) % self.dp
        pp_i = rank // (tp * self.dp)
        return dict(tp=tp_i, dp=dp_i, pp=pp_i, wp=dp_i % wp, wdp=dp_i // wp)

    def _group_lists(self) -> Dict[ParallelMode, List[List[int]]]:
        ws, tp, wp, pp, dp = self.world_size, self.cfg.tensor, self.cfg.weight, self.cfg.pipeline, self.dp
        by = lambda key: self._partition(key)
        out = {ParallelMode.GLOBAL: [list(range(ws))]}
        out[ParallelMode.TENSOR] = by(lambda c: (c["pp"], c["dp"]))
        out[ParallelMode.DATA] = by(lambda c: (c["pp"], c["tp"]))
        out[ParallelMode.PIPELINE] = by(lambda c: (c["dp"], c["tp"]))
        out[ParallelMode.WEIGHT] = by(lambda c: (c["pp"], c["wdp"], c["tp"]))
        out[ParallelMode.WEIGHT_DATA] = by(lambda c: (c["pp"], c["wp"], c["tp"]))
        out[ParallelMode.COMMON_DATA] = by(lambda c: (c["pp"], c["wdp"]))
        base = ParallelMode.WEIGHT_DATA if wp > 1 else ParallelMode.DATA
        out[ParallelMode.ZERO1] = [g[i:i + self.zero1] for g in out[base] for i in range(0, len(g), self.zero1)]
        ep, ewp = max(self.cfg.expert, 1), max(self.cfg.expert_weight, 1)
        stage = lambda p: [r for r in range(ws) if self.coords(r)["pp"] == p]
        out[ParallelMode.EXPERT], out[ParallelMode.EXPERT_DATA], out[ParallelMode.EXPERT_WEIGHT] = [], [], []
        for p_i in range(pp):
            rs = stage(p_i)
            # expert-weight is the fastest axis inside a stage, then expert, then expert-data
            n = len(rs)
            edp = n // (ep * ewp)
            for d in range(edp):
                for w in range(ewp):
                    out[ParallelMode.EXPERT].append([rs[(d * ep + e) * ewp + w] for e in range(ep)])
            for e in range(ep):
                for w in range(ewp):
                    out[ParallelMode.EXPERT_DATA].append([rs[(d * ep + e) * ewp + w] for d in range(edp)])
            for d in range(edp):
                for e in range(ep):
                    out[ParallelMode.EXPERT_WEIGHT].append([rs[(d * ep + e) * ewp + w] for w in range(ewp)])
        ez = self.cfg.expert_zero1
        out[ParallelMode.EXPERT_ZERO1] = []
        for g in out[ParallelMode.EXPERT_DATA]:
            z = len(g) if ez in (-1, 0) else ez
            out[ParallelMode.EXPERT_ZERO1] += [g[i:i + z] for i in range(0, len(g), z)]
        return out

    def _partition(self, key) -> List[List[int]]:
        d: Dict[tuple, List[int]] = {}
        for r in range(self.world_size):
            d.setdefault(key(self.coords(r)), []).append(r)
        return [d[k] for k in sorted(d)]

    def _build(self, create_groups: bool, backend: Optional[str]):
        for mode, lists in self._group_lists().items():
            for ranks in lists:
                grp = None
                if create_groups and dist.is_initialized() and len(ranks) > 1 and mode != ParallelMode.GLOBAL:
                    grp = dist.new_group(ranks, backend=backend)     # every rank creates every group
                if self.rank in ranks:
                    self.ranks_in_group[mode] = ranks
                    self.sizes[mode] = len(ranks)
                    self.local_rank[mode] = ranks.index(self.rank)
                    self.groups[mode] = grp if mode != ParallelMode.GLOBAL else (dist.group.WORLD if dist.is_initialized() else None)

    # ---- queries (the subset of the reference's gpc API the framework uses) ----
    def get_world_size(self, mode: ParallelMode) -> int:
        return self.sizes.get(mode, 1)

    def get_local_rank(self, mode: ParallelMode) -> int:
        return self.local_rank.get(mode, 0)

    def get_group(self, mode: ParallelMode):
        return self.groups.get(mode)

    def get_ranks_in_group(self, mode: ParallelMode) -> List[int]:
        return self.ranks_in_group.get(mode, [self.rank])

    def is_pipeline_first_stage(self) -> bool:
        return self.get_local_rank(ParallelMode.PIPELINE) == 0

    def is_pipeline_last_stage(self) -> bool:
        return self.get_local_rank(ParallelMode.PIPELINE) == self.get_world_size(ParallelMode.PIPELINE) - 1

    def is_using_isp(self) -> bool:
        return self.cfg.tensor_mode == "isp"

    def seed_for(self, base_seed: int, mode: ParallelMode) -> int:
        """Per-mode RNG seed: equal inside replicas of a mode, distinct across its shards
        (reference: core/context/parallel_context.py:754-803, random.py)."""
        c = self.coords(self.rank)
        if mode == ParallelMode.DATA:
            return base_seed + 1024 * c["dp"] + 7 * c["pp"]
        if mode == ParallelMode.TENSOR:
            return base_seed + 1024 * c["dp"] + 7 * c["pp"] + 131 * (c["tp"] + 1)
        if mode == ParallelMode.WEIGHT:
            return base_seed + 1024 * c["wdp"] + 7 * c["pp"] + 257 * (c["wp"] + 1)
        return base_seed


def init_distributed(backend: str = "nccl", timeout_s: Optional[int] = None, device=None) -> None:
    """``torch.distributed`` rendezvous from torchrun's environment (RANK, WORLD_SIZE, MASTER_*).
    The collective timeout follows the reference's NCCL_TIMEOUT convention (utils/timeout.py:59-64)."""
    if dist.is_initialized():
        return
    t = int(os.environ.get("NCCL_TIMEOUT", timeout_s or 1800))
    kw = {}
    if device is not None and backend == "nccl":
        kw["device_id"] = device
    dist.init_process_group(backend, timeout=timedelta(seconds=t), **kw)
