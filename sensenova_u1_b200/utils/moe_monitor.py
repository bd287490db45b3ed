"""Expert-load statistics of the MoE layers.

Collects, per layer and mixture (understanding / generation), how many token copies each expert
received in the last step, and derives the numbers the reference's monitor logs
(training/sensenovalm/model/moe/monitor/moe_monitor.py:20-142): the fraction of token copies above
the uniform share ("overflow" that a capacity-based router would drop), the number of experts that
received nothing, the max/mean load ratio and the entropy of the load distribution.  Counts stay on
the device while the step runs (one small tensor per layer, no synchronisation); ``summary`` reduces
them over the data-parallel group and reads them back once.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch


class MoEMonitor:
    def __init__(self, group=None, ep_size: int = 1):
        """``ep_size`` > 1 also reports the load per expert-parallel rank (experts are split evenly,
        in order, over the ranks): the slowest rank sets the step time."""
        self.group = group
        self.ep_size = ep_size
        self.counts: Dict[Tuple[int, str], torch.Tensor] = {}
        self.enabled = True

    def record(self, layer: int, mixture: str, counts: torch.Tensor) -> None:
        """``counts`` [E] int32: token copies per expert of this rank's batch (device tensor)."""
        if not self.enabled:
            return
        key = (layer, mixture)
        c = counts.detach().to(torch.float32)
        if key in self.counts and self.counts[key].shape == c.shape:
            self.counts[key].add_(c)
        else:
            self.counts[key] = c.clone()

    def reset(self) -> None:
        self.counts.clear()

    @staticmethod
    def load_stats(load: torch.Tensor, ep_size: int = 1) -> Dict[str, float]:
        """Statistics of one load vector (any device, float)."""
        load = load.double()
        tot = float(load.sum())
        E = load.numel()
        if tot <= 0:
            return {"tokens": 0.0, "above_avg_frac": 0.0, "idle_experts": float(E), "max_over_mean": 0.0, "entropy": 0.0}
        extra = {}
        if ep_size > 1 and E % ep_size == 0:
            per_rank = load.view(ep_size, E // ep_size).sum(dim=1)
            extra["rank_max_over_mean"] = float(per_rank.max()) / (tot / ep_size)
        mean = tot / E
        p = load / tot
        ent = float(-(p[p > 0] * p[p > 0].log()).sum()) / math.log(E) if E > 1 else 1.0
        return {**extra, "tokens": tot,
                "above_avg_frac": float((load - mean).clamp_min(0).sum()) / tot,
                "idle_experts": float((load == 0).sum()),
                "max_over_mean": float(load.max()) / mean,
                "entropy": ent}

    def summary(self, reduce: bool = True) -> Dict[str, float]:
        """Per layer/mixture statistics plus their means, as flat scalar names for the metric writer."""
        import torch.distributed as dist
        out: Dict[str, float] = {}
        if not self.counts:
            return out
        keys = sorted(self.counts)
        agg: Dict[str, list] = {}
        for key in keys:
            c = self.counts[key]
            if reduce and dist.is_available() and dist.is_initialized():
                c = c.clone()
                dist.all_reduce(c, group=self.group)
            st = self.load_stats(c.cpu(), self.ep_size)
            for name, v in st.items():
                out[f"moe/{key[1]}/layer{key[0]}/{name}"] = v
                agg.setdefault(f"moe/{key[1]}/mean_{name}", []).append(v)
        for name, vs in agg.items():
            out[name] = sum(vs) / len(vs)
        return out
