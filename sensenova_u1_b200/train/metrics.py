"""Per-step training metrics, throughput statistics (tgs), timers and writers.

``tgs`` = tokens in the batch x data-parallel size / global world size / step time, the
reference's throughput definition (training/sensenovavl/train/record_metrics.py:363-421), with
its running aggregates (last 1 / 10 / 50, average, simple moving average).  Writers: JSON lines
always, TensorBoard when the package is importable (utils/writer.py:30-242).
"""
from __future__ import annotations

import json
import os
import time
from collections import deque
from contextlib import contextmanager
from pathlib import Path
from typing import Dict, Optional


class ThroughputStats:
    def __init__(self):
        self.hist = deque(maxlen=50)
        self.total_tokens = 0
        self.total_time = 0.0
        self.sma = None

    def update(self, tokens_in_batch: int, dp_world: int, global_world: int, seconds: float) -> Dict[str, float]:
        tgs = tokens_in_batch * dp_world / global_world / max(seconds, 1e-9)
        self.hist.append(tgs)
        self.total_tokens += tokens_in_batch * dp_world / global_world
        self.total_time += seconds
        self.sma = tgs if self.sma is None else 0.9 * self.sma + 0.1 * tgs
        h = list(self.hist)
        return {"tgs": tgs, "tgs/last_tgs_1": tgs, "tgs/last_tgs_10": sum(h[-10:]) / len(h[-10:]),
                "tgs/last_tgs_50": sum(h) / len(h), "tgs/tgs_avg": self.total_tokens / self.total_time,
                "tgs/tgs_SMA": self.sma}


class Timers:
    """Named wall-clock timers; ``sync=True`` synchronises the device around the region
    (reference: utils/megatron_timers.py)."""

    def __init__(self):
        self.t: Dict[str, float] = {}

    @contextmanager
    def __call__(self, name: str, sync: bool = False):
        if sync:
            import torch
            if torch.cuda.is_available():
                torch.cuda.synchronize()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if sync:
                import torch
                if torch.cuda.is_available():
                    torch.cuda.synchronize()
            self.t[name] = self.t.get(name, 0.0) + time.perf_counter() - t0

    def pop(self) -> Dict[str, float]:
        out, self.t = self.t, {}
        return out


class Writer:
    def __init__(self, run_dir: str, rank: int = 0, enable_tb: bool = True):
        self.dir = Path(run_dir)
        self.rank = rank
        self.jsonl = None
        self.tb = None
        if rank == 0:
            (self.dir / "logs").mkdir(parents=True, exist_ok=True)
            self.jsonl = open(self.dir / "logs" / "metrics.jsonl", "a")
            if enable_tb:
                try:
                    from torch.utils.tensorboard import SummaryWriter
                    self.tb = SummaryWriter(str(self.dir / "tensorboards"))
                except Exception:
                    self.tb = None

    def add_scalars(self, scalars: Dict[str, float], step: int):
        if self.jsonl is None:
            return
        self.jsonl.write(json.dumps({"step": step, **{k: float(v) for k, v in scalars.items()}}) + "\n")
        self.jsonl.flush()
        if self.tb is not None:
            for k, v in scalars.items():
                self.tb.add_scalar(k, float(v), step)

    def close(self):
        if self.jsonl:
            self.jsonl.close()
        if self.tb:
            self.tb.close()


def format_line(step: int, m: Dict[str, float]) -> str:
    keys = ["loss", "ce", "fm", "mtp", "moe_aux", "lr", "grad_norm", "tgs", "tgs/tgs_avg", "step_time"]
    return f"step={step} " + " ".join(f"{k}={m[k]:.4g}" for k in keys if k in m)
