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


def step_tflops(cfg, tokens: int, seconds: float, world: int = 1, recompute: bool = True,
                attention_pairs: Optional[float] = None) -> Dict[str, float]:
    """Achieved TFLOP/s per GPU of one training step (the reference logs the Megatron estimate,
    training/sensenovalm/utils/common.py:209-247: 3 passes, 4 with activation checkpointing, over
    ``(8 + 4 * 1.5 * mlp_ratio) * tokens * hidden^2`` per layer, ``4 * tokens * seq * hidden`` of attention and the
    vocabulary head).  This form counts what this model actually multiplies: grouped-query projections
    (``q_dim + 2 * kv_dim`` columns), the SwiGLU FFN (or the routed experts' share for MoE), one branch per
    token, and attention over the allowed (query, key) pairs when ``attention_pairs`` is given (dense causal
    ``tokens^2 / 2`` otherwise).  ``tflops`` excludes the recomputation, ``tflops_hw`` includes it."""
    H, L = cfg.hidden_size, cfg.num_layers
    proj = H * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * H
    if getattr(cfg, "is_moe", False):
        ffn = 3 * H * cfg.moe_intermediate_size * cfg.num_experts_per_tok + H * cfg.num_experts
    else:
        ffn = 3 * H * cfg.ffn_size
    pairs = float(attention_pairs) if attention_pairs is not None else tokens * tokens / 2.0
    fwd = 2.0 * tokens * (proj + ffn) * L + 4.0 * pairs * cfg.q_dim * L + 2.0 * tokens * H * cfg.vocab_size
    model = 3.0 * fwd
    hw = model + (fwd - 2.0 * tokens * H * cfg.vocab_size if recompute else 0.0)
    denom = max(seconds, 1e-9) * max(world, 1) * 1e12
    return {"tflops": model / denom, "tflops_hw": hw / denom}


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
    """Scalars of the reporting rank: ``logs/metrics.jsonl`` and TensorBoard events.  ``tensorboard_folder`` (config key
    or environment variable of the same name) puts the events somewhere else; ``resume_tb_folder`` continues the event
    files of an earlier run by writing into that folder (initialize/launch.py:316-326, utils/writer.py:30-96)."""

    def __init__(self, run_dir: str, rank: int = 0, enable_tb: bool = True, tensorboard_folder: Optional[str] = None,
                 resume_tb_folder: Optional[str] = None, report_rank: int = 0):
        self.dir = Path(run_dir)
        self.rank = rank
        self.jsonl = None
        self.tb = None
        if rank == report_rank:
            (self.dir / "logs").mkdir(parents=True, exist_ok=True)
            self.jsonl = open(self.dir / "logs" / "metrics.jsonl", "a")
            if enable_tb:
                tb_dir = resume_tb_folder or tensorboard_folder or str(self.dir / "tensorboards")
                try:
                    from torch.utils.tensorboard import SummaryWriter
                    self.tb = SummaryWriter(tb_dir)
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


class RankLog:
    """Text log of one rank: every line goes to ``<run_dir>/logs/rank<r>.log`` with a time stamp, and to the console on
    the rank that reports (the reference writes a file per rank under ``RUN/<job>/<time>/logs`` and echoes on the
    logging rank: utils/logger.py:1-72)."""

    def __init__(self, run_dir: str, rank: int = 0, echo: bool = True):
        self.echo = echo
        d = Path(run_dir) / "logs"
        try:
            d.mkdir(parents=True, exist_ok=True)
            self.f = open(d / f"rank{rank}.log", "a", encoding="utf-8")
        except OSError:
            self.f = None                      # a read-only run directory must not stop the job

    def __call__(self, line: str, echo: Optional[bool] = None) -> None:
        if self.f is not None:
            self.f.write(time.strftime("%Y-%m-%d %H:%M:%S ") + line + "\n")
            self.f.flush()
        if self.echo if echo is None else echo:
            print(line, flush=True)

    def close(self) -> None:
        if self.f is not None:
            self.f.close()
            self.f = None


TASK_NAMES = {3: "t2i", 4: "editing", 5: "interleave"}      # generation task ids of the data pipeline


class AccPerplex:
    """Token accuracy and perplexity, overall and per dataset type (reference: ``AccPerplex``,
    training/sensenovalm/model/metrics.py:81-300).  Fed with sums (correct predictions, label rows, loss x rows),
    which the loss kernel already produces; ranks' sums are added with one all-reduce of a small vector."""

    def __init__(self, dataset_types=("all",), group=None):
        self.types = list(dataset_types)
        self.group = group
        self.reset()

    def reset(self):
        self.sums = {t: [0.0, 0.0, 0.0] for t in self.types}        # correct, rows, loss sum

    def update(self, correct: float, rows: float, loss_sum: float, dataset_type: str = "all"):
        s = self.sums.setdefault(dataset_type, [0.0, 0.0, 0.0])
        s[0] += float(correct); s[1] += float(rows); s[2] += float(loss_sum)
        if dataset_type != "all" and "all" in self.sums:
            a = self.sums["all"]
            a[0] += float(correct); a[1] += float(rows); a[2] += float(loss_sum)

    def get_metric(self, reset: bool = True) -> Dict[str, float]:
        import math
        import torch
        import torch.distributed as dist
        keys = sorted(self.sums)
        t = torch.tensor([v for k in keys for v in self.sums[k]], dtype=torch.float64)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            if dist.get_backend(self.group) == "nccl":
                t = t.cuda()
            dist.all_reduce(t, group=self.group)
            t = t.cpu()
        out = {}
        for i, k in enumerate(keys):
            c, r, l = t[3 * i:3 * i + 3].tolist()
            if r > 0:
                sfx = "" if k == "all" else f"/{k}"
                out["acc" + sfx] = c / r
                out["perplexity" + sfx] = math.exp(min(l / r, 50.0))
                out["tokens" + sfx] = r
        if reset:
            self.reset()
        return out


class TrainRecord:
    """Running counters of a training job (reference: training/sensenovavl/train/record_metrics.py:95-239, 431-481):
    consumed tokens / text tokens / images / generated images / samples, generation samples per task, padding
    tokens, skipped non-finite steps; ``update`` takes the step's host batches and returns the flat dict to log."""

    FIELDS = ("num_consumed_tokens", "num_consumed_text_tokens", "num_consumed_images", "num_consumed_gen_images",
              "num_consumed_samples", "num_gen_samples_t2i", "num_gen_samples_editing", "num_gen_samples_interleave",
              "num_padding_tokens")

    def __init__(self, dp_world: int = 1, group=None):
        self.dp_world, self.group = dp_world, group
        self.c = {k: 0 for k in self.FIELDS}

    @staticmethod
    def count(batches) -> Dict[str, int]:
        import torch
        from ..data.batch import KIND_GEN_IMG, KIND_PAD, KIND_TEXT, KIND_UND_IMG
        out = {k: 0 for k in TrainRecord.FIELDS}
        for b in batches:
            kind = b.kind
            out["num_consumed_tokens"] += int(b.n_tokens)
            out["num_consumed_text_tokens"] += int((kind == KIND_TEXT).sum())
            out["num_padding_tokens"] += int((kind == KIND_PAD).sum())
            out["num_consumed_samples"] += int(b.n_samples)
            img = b.meta[:, 2]
            und_ids = torch.unique(b.meta[kind == KIND_UND_IMG][:, [0, 2]], dim=0).shape[0] if (kind == KIND_UND_IMG).any() else 0
            gen_rows = b.meta[kind == KIND_GEN_IMG]
            gen_ids = torch.unique(gen_rows[:, [0, 2]], dim=0) if gen_rows.numel() else gen_rows[:, :2]
            out["num_consumed_images"] += int(und_ids) + int(gen_ids.shape[0])
            out["num_consumed_gen_images"] += int(gen_ids.shape[0])
            if b.gen_task.numel():
                # one generation sample = one (document, task) pair that owns generated tokens
                docs = b.meta[b.gen_rows.cpu() if b.gen_rows.is_cuda else b.gen_rows][:, 0]
                pairs = torch.unique(torch.stack([docs.cpu().long(), b.gen_task.cpu().long()], 1), dim=0)
                for tid, name in TASK_NAMES.items():
                    out[f"num_gen_samples_{name}"] += int((pairs[:, 1] == tid).sum())
        return out

    def update(self, batches, skipped_steps: int = 0) -> Dict[str, float]:
        import torch
        import torch.distributed as dist
        local = self.count(batches)
        self.last = local                          # this rank's counts of the step (padding-free throughput)
        keys = list(self.FIELDS)
        t = torch.tensor([local[k] for k in keys], dtype=torch.float64)
        if self.dp_world > 1 and dist.is_initialized():
            if dist.get_backend(self.group) == "nccl":
                t = t.cuda()
            dist.all_reduce(t, group=self.group)
            t = t.cpu()
        for k, v in zip(keys, t.tolist()):
            self.c[k] += int(v)
        out = dict(self.c)
        out["inf_nan_skip_batches"] = int(skipped_steps)
        return out

    def state_dict(self):
        return dict(self.c)

    def load_state_dict(self, sd):
        self.c.update({k: int(v) for k, v in sd.items() if k in self.c})


class WandbWriter:
    """Optional Weights & Biases sink for the keys that contain "loss" (reference: utils/writer.py:191-201).  Active
    only when the ``wandb`` package is importable and ``WANDB_PROJECT`` (or ``project``) is given; never a
    hard dependency."""

    def __init__(self, project: Optional[str] = None, name: Optional[str] = None, rank: int = 0):
        self.run = None
        project = project or os.environ.get("WANDB_PROJECT")
        if rank != 0 or not project:
            return
        try:
            import wandb
            self.run = wandb.init(project=project, name=name or os.environ.get("WANDB_NAME"),
                                  mode=os.environ.get("WANDB_MODE", "offline"))
        except Exception:
            self.run = None

    def add_scalars(self, scalars: Dict[str, float], step: int):
        if self.run is not None:
            self.run.log({k: float(v) for k, v in scalars.items() if "loss" in k}, step=step)

    def close(self):
        if self.run is not None:
            self.run.finish()


def format_line(step: int, m: Dict[str, float]) -> str:
    keys = ["loss", "ce", "fm", "image_gen_loss_t2i", "image_gen_loss_editing", "image_gen_loss_interleave", "mtp",
            "moe_aux", "acc", "perplexity", "lr", "grad_norm", "tgs", "tgs/tgs_avg", "step_time", "num_consumed_tokens"]
    return f"step={step} " + " ".join(f"{k}={m[k]:.4g}" for k in keys if k in m)
