"""Learning-rate and beta2 schedules
(reference: training/sensenovalm/solver/schedulers/lr_scheduler.py:13-135, beta2_scheduler.py:9-35)."""
from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass
class FineTuneCosineAnnealingWarmupLR:
    """``init_steps`` steps at lr 0, linear warm-up over ``warmup_ratio * total_steps`` steps, then
    cosine decay to ``eta_min * base_lr`` (or a constant lr when ``kind == 'constant'``)."""
    base_lr: float
    total_steps: int
    init_steps: int = 0
    warmup_ratio: float = 0.0
    eta_min: float = 0.0          # ratio of base_lr
    kind: str = "cosine"
    offset: int = 0
    last_epoch: int = -1

    def lr_at(self, step: int) -> float:
        step = step + self.offset
        if step < self.init_steps:
            return 0.0
        s = step - self.init_steps
        total = max(self.total_steps - self.init_steps, 1)
        warm = int(self.warmup_ratio * total)
        if s < warm:
            return self.base_lr * (s + 1) / warm
        if self.kind == "constant":
            return self.base_lr
        prog = min(1.0, (s - warm) / max(total - warm, 1))
        lo = self.eta_min * self.base_lr
        return lo + (self.base_lr - lo) * 0.5 * (1 + math.cos(math.pi * prog))

    def step(self) -> float:
        self.last_epoch += 1
        return self.lr_at(self.last_epoch)

    def state_dict(self):
        return {"last_epoch": self.last_epoch}

    def load_state_dict(self, sd):
        self.last_epoch = int(sd["last_epoch"])


@dataclass
class Beta2Scheduler:
    """beta2_t = max(init_beta2, 1 - t^-c) when c > 0, else constant."""
    init_beta2: float = 0.95
    c: float = 0.0
    cur_iter: int = -1

    def step(self) -> float:
        self.cur_iter += 1
        if self.c <= 0 or self.cur_iter <= 0:
            return self.init_beta2
        return max(self.init_beta2, 1 - self.cur_iter ** (-self.c))
