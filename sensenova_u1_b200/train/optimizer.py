"""ZeRO-1 AdamW over the flat parameter arenas.

Each data-parallel rank owns one contiguous range of every arena: it receives the
sum of the gradients of that range (reduce-scatter), updates the fp32 master of the
range with the fused unscale + clip + AdamW kernel, and the updated bf16 weights are
all-gathered back in place.  This is the reduce-scatter / all-gather form of the
reference's ZeRO-1, which all-reduces full gradients and then broadcasts every
partition (training/sensenovalm/solver/optimizer/hybrid_zero_optim.py:626-690,
832-1070) at twice the wire traffic; the update itself is numerically the same.

On CPU tensors (gloo tests) the same schedule runs with a PyTorch AdamW on an fp32
master of the shard.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..models.params import ParamStore


@dataclass
class AdamConfig:
    lr: float = 2e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.0
    clip_grad_norm: float = 1.0
    state_dtype: str = "auto"      # "fp32" | "bf16" | "auto" (fp32 when it fits in device memory)
    lr_scale: Optional[Dict[str, float]] = None   # per role: vit, llm, fm_modules, embed, ...


class ZeroAdamW:
    def __init__(self, store: ParamStore, cfg: AdamConfig, group=None, grad_divisor: float = 1.0):
        self.store, self.cfg, self.group = store, cfg, group
        self.world = dist.get_world_size(group) if (dist.is_initialized() and group is not False) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.grad_divisor = grad_divisor
        self.step_count = 0
        self.dev = store.device
        self.cuda = self.dev.type == "cuda"
        self.lr = cfg.lr
        self.shard: Dict[str, Tuple[int, int]] = {}
        self.state: Dict[str, Dict[str, torch.Tensor]] = {}
        total_shard = 0
        for a, n in store.sizes.items():
            if n % self.world:
                raise ValueError(f"arena {a} ({n}) does not divide over {self.world} ranks")
            per = n // self.world
            self.shard[a] = (self.rank * per, (self.rank + 1) * per)
            total_shard += per
        sd = cfg.state_dtype
        if sd == "auto":
            sd = "fp32"
            if self.cuda:
                free, _ = torch.cuda.mem_get_info(self.dev)
                need = total_shard * (2 + 8) + (4 << 30)
                if need > free:
                    sd = "bf16"
        self.state_dtype = torch.float32 if sd == "fp32" else torch.bfloat16
        for a, (lo, hi) in self.shard.items():
            n = hi - lo
            st = {"m": torch.zeros(n, dtype=self.state_dtype, device=self.dev),
                  "v": torch.zeros(n, dtype=self.state_dtype, device=self.dev)}
            if self.cuda:
                st["lo"] = torch.zeros(n, dtype=torch.int16, device=self.dev)
            else:
                st["master"] = store.arena[a][lo:hi].float().clone()
            self.state[a] = st
        self.norm_sq = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self.skipped = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.ranges = {a: self._ranges(a) for a in store.sizes}

    def _ranges(self, arena) -> List[Tuple[int, int, float, float]]:
        """Merged (start, end, lr_scale, weight_decay) runs of the shard, arena coordinates."""
        lo, hi = self.shard[arena]
        scales = self.cfg.lr_scale or {}
        runs: List[List] = []
        pos = 0
        for s, e, spec in self.store.segments(arena):
            wd = self.cfg.weight_decay if spec.decay else 0.0
            sc = scales.get(spec.role, 1.0)
            if runs and runs[-1][2] == sc and runs[-1][3] == wd:
                runs[-1][1] = e
            else:
                runs.append([pos, e, sc, wd])   # the alignment gap before a tensor joins its run
            pos = e
        if runs:
            runs[-1][1] = self.store.sizes[arena]
        out = []
        for s, e, sc, wd in runs:
            s2, e2 = max(s, lo), min(e, hi)
            if e2 > s2:
                out.append((s2, e2, sc, wd))
        return out

    # ------------------------------------------------------------------ step
    def reduce_gradients(self):
        """Sum of gradients over data-parallel ranks lands in each rank's own shard."""
        if self.world == 1:
            return
        for a, (lo, hi) in self.shard.items():
            g = self.store.grad_arena[a]
            if self.cuda:
                dist.reduce_scatter_tensor(g[lo:hi], g, op=dist.ReduceOp.SUM, group=self.group)
            else:
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.group)

    def grad_norm_sq(self) -> torch.Tensor:
        self.norm_sq.zero_()
        for a, (lo, hi) in self.shard.items():
            g = self.store.grad_arena[a][lo:hi]
            if self.cuda:
                from ..ops import fused
                fused.sumsq(g, self.norm_sq)
            else:
                self.norm_sq += g.float().pow(2).sum()
        if self.world > 1:
            dist.all_reduce(self.norm_sq, op=dist.ReduceOp.SUM, group=self.group)
        return self.norm_sq

    def step(self, lr: Optional[float] = None) -> None:
        c = self.cfg
        lr = self.lr if lr is None else lr
        self.step_count += 1
        self.reduce_gradients()
        nsq = self.grad_norm_sq()
        pre = 1.0 / self.grad_divisor
        if self.cuda:
            from ..ops import fused
            for a, (lo, hi) in self.shard.items():
                st = self.state[a]
                P, G = self.store.arena[a], self.store.grad_arena[a]
                for s, e, sc, wd in self.ranges[a]:
                    fused.adamw(P[s:e], st["lo"][s - lo:e - lo], G[s:e], st["m"][s - lo:e - lo],
                                st["v"][s - lo:e - lo], lr=lr * sc, beta1=c.beta1, beta2=c.beta2,
                                eps=c.eps, weight_decay=wd, step=self.step_count, grad_prescale=pre,
                                norm_sq=nsq, max_norm=c.clip_grad_norm, skipped=self.skipped)
        else:
            norm = float(nsq.sqrt()) * pre
            if not math.isfinite(norm):
                self.skipped += 1
            else:
                coef = min(1.0, c.clip_grad_norm / (norm + 1e-6)) if c.clip_grad_norm > 0 else 1.0
                bc1 = 1 - c.beta1 ** self.step_count
                bc2 = 1 - c.beta2 ** self.step_count
                for a, (lo, hi) in self.shard.items():
                    st = self.state[a]
                    for s, e, sc, wd in self.ranges[a]:
                        g = self.store.grad_arena[a][s:e].float() * (pre * coef)
                        m, v, w = st["m"][s - lo:e - lo], st["v"][s - lo:e - lo], st["master"][s - lo:e - lo]
                        m.mul_(c.beta1).add_(g, alpha=1 - c.beta1)
                        v.mul_(c.beta2).addcmul_(g, g, value=1 - c.beta2)
                        w.mul_(1 - lr * sc * wd)
                        w.addcdiv_(m.float(), (v.float().sqrt() / math.sqrt(bc2)).add_(c.eps), value=-lr * sc / bc1)
                        self.store.arena[a][s:e] = w.to(self.store.dtype)
        self.gather_params()

    def gather_params(self):
        if self.world == 1:
            return
        for a, (lo, hi) in self.shard.items():
            P = self.store.arena[a]
            dist.all_gather_into_tensor(P, P[lo:hi].clone() if not self.cuda else P[lo:hi], group=self.group)

    # ------------------------------------------------------------ checkpoint
    def state_dict(self):
        return {"step": self.step_count, "lr": self.lr, "shard": dict(self.shard), "world": self.world,
                "state": {a: {k: v.cpu() for k, v in st.items()} for a, st in self.state.items()}}

    def load_state_dict(self, sd):
        if sd["world"] != self.world:
            raise ValueError(f"optimizer shards were saved with zero size {sd['world']}, now {self.world}")
        self.step_count = sd["step"]
        self.lr = sd.get("lr", self.lr)
        for a, st in sd["state"].items():
            for k, v in st.items():
                self.state[a][k].copy_(v)
