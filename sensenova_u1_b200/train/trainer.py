"""Single-process-per-GPU SFT trainer: host batch -> device -> forward/backward ->
ZeRO-1 AdamW step -> loss.  The public call a user makes is :meth:`Trainer.train_step`.

Reference flow: TrainerBuilder.fit / _process_batch
(training/sensenovalm/core/trainer_builder.py:453-689), NonPipelineScheduler
(core/scheduler/no_pipeline_scheduler.py:132-340), Engine.step (core/engine.py:134-157).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..config import ModelConfig
from ..data.batch import PackedBatch
from ..models.params import ParamStore
from .optimizer import AdamConfig, PeerZeroAdamW, ZeroAdamW


class Trainer:
    def __init__(self, cfg: ModelConfig, store: ParamStore, adam: Optional[AdamConfig] = None,
                 dp_group=None, host_group=None, grad_accum: int = 1, ema_decay: float = 0.0,
                 comm: str = "nccl", ep_group=None, max_tokens: int = 16384, ep_capacity_factor: Optional[float] = None,
                 cp_group=None, tp_group=None):
        """``tp_group``: tensor-parallel group; ``cfg`` / ``store`` are then the local slice
        (parallel/tensor_engine.py: ``tp_local_config``, ``shard_store_tp``), every rank of the group must be given
        the same batches, and ``dp_group`` is the group of the ranks that hold the same slice."""
        self.cfg, self.store = cfg, store
        self.dev = store.device
        if tp_group is not None and dp_group is None and dist.is_initialized():
            # data-parallel group = the ranks that hold the same tensor-parallel slice (tensor-parallel ranks are
            # consecutive); every rank creates every group, as torch.distributed requires
            t, w, me = dist.get_world_size(tp_group), dist.get_world_size(), dist.get_rank()
            for j in range(t):
                grp = dist.new_group(list(range(j, w, t)))
                if me % t == j:
                    dp_group = grp
        self.dp_world = dist.get_world_size(dp_group) if dist.is_initialized() else 1
        self.dp_group, self.host_group = dp_group, host_group
        self.grad_accum = grad_accum
        if self.dev.type == "cuda":
            if cfg.is_moe:
                from ..models.engine_moe import MoEMoTEngine as Eng
            else:
                from ..models.engine import MoTEngine as Eng
            if cfg.is_moe and cfg.ep_size > 1:
                # experts split over the ranks of ep_group (default: the data-parallel group);
                # rows are exchanged through peer memory (parallel/expert.py)
                from ..parallel.expert import ExpertParallel
                ep = ExpertParallel(ep_group if ep_group is not None else dp_group, self.dev, cfg.hidden_size,
                                    {"gen": (cfg.gen_num_experts, cfg.gen_num_experts_per_tok),
                                     "und": (cfg.num_experts, cfg.num_experts_per_tok)},
                                    max_tokens, ep_capacity_factor)
                self.engine = Eng(cfg, store, ep=ep)
            else:
                self.engine = Eng(cfg, store)
            if cp_group is not None:
                # one packed sequence split over the ranks of cp_group (data/batch.split_context_parallel
                # cuts the batch); weights stay replicated, so gradients are reduced exactly as in data parallel
                from ..parallel.context_attention import ContextParallelAttention
                self.engine.cp = ContextParallelAttention(cp_group, self.dev, max_tokens, cfg.num_heads,
                                                          cfg.num_kv_heads)
            if tp_group is not None and dist.get_world_size(tp_group) > 1:
                if cfg.num_mtp_layers > 0 or cfg.is_moe:
                    raise NotImplementedError("tensor parallel is built for the dense decoder stack without "
                                              "multi-token-prediction heads")
                from ..parallel.tensor_engine import PeerAllReduce
                self.engine.tp = PeerAllReduce(tp_group, self.dev, max_tokens * cfg.hidden_size)
        else:
            self.engine = None
        # gradients are summed over ranks and micro-batches; the loss normalisers already
        # average over data-parallel ranks, so divide by the number of ranks only
        # comm="peer": reduce-scatter / all-gather done by this package's kernels over NVLink peer
        # memory (arenas must be symmetric); comm="nccl": the NCCL collectives (baseline)
        self.wp = None
        from ..parallel.weight_parallel import WeightParallelStore
        if isinstance(store, WeightParallelStore):
            # weight parallel: weights, gradients and optimizer state sharded 1/N; layers gathered on demand
            from ..parallel.weight_parallel import WeightParallelAdamW
            self.optim = self.wp = WeightParallelAdamW(store, adam or AdamConfig(), group=dp_group,
                                                       grad_divisor=float(self.dp_world))
        elif comm == "peer" and self.dp_world > 1 and self.dev.type == "cuda":
            if store.symm is None:
                from ..parallel.symm import symmetric_arenas
                symmetric_arenas(store, dp_group)
                if self.engine is not None:
                    self.engine.p, self.engine.g = store.p, store.g
            self.optim = PeerZeroAdamW(store, adam or AdamConfig(), group=dp_group, grad_divisor=float(self.dp_world))
        else:
            self.optim = ZeroAdamW(store, adam or AdamConfig(), group=dp_group, grad_divisor=float(self.dp_world))
        self.step_idx = 0
        self.ema = None
        self.ema_decay = ema_decay
        if ema_decay > 0:
            # fp32 shadow of the pieces this rank updates (the reference averages its local shards the same way,
            # core/model_average.py:182-250); weight parallel: the matrix piece is the rank's shard
            self.ema = {a: (store.shard.tensor[: self.optim.state[a]["m"].numel()].float() if (self.wp is not None and a == "mat")
                            else torch.cat([store.arena[a][p[3]:p[4]].float() for p in lst]))
                        for a, lst in self.optim.pieces.items()}
        if self.engine is not None:
            self.engine.on_grads_ready = self._grads_ready
            self.engine.on_weights_needed = self._weights_needed
            if self.wp is not None:
                self.engine.on_backward_begin = self.wp.begin_micro_backward
                self.engine.on_layer_backward_begin = self._wp_layer_backward
        self._last_micro = True
        self.profile_events = None      # set to a list to collect CUDA events around every optimizer step

    # ---------------------------------------------------------------------
    def _normalisers(self, batches: Sequence[PackedBatch]):
        ce = sum(b.ce_weight_sum for b in batches)
        gn = sum(b.gen_weight_sum for b in batches)
        if self.dp_world > 1:
            t = torch.tensor([ce, gn], dtype=torch.float64)
            if self.host_group is not None:
                dist.all_reduce(t, group=self.host_group)
            else:
                t = t.to(self.dev)
                dist.all_reduce(t, group=self.dp_group)
                t = t.cpu()
            ce, gn = (t / self.dp_world).tolist()
        return max(ce, 1e-12), max(gn, 1.0)

    def train_step(self, host_batches: Sequence[PackedBatch], lr: Optional[float] = None) -> Dict[str, float]:
        """One optimizer step over ``grad_accum`` micro-batches given as host (pinned) batches.
        Copies them to the device, runs the step and reads the loss back."""
        dev_batches = [b.to(self.dev, non_blocking=True) for b in host_batches]
        out = self.step_on_device(dev_batches, lr=lr)
        return {k: float(v) for k, v in out.items()}       # device -> host read of the results

    def step_on_device(self, batches: Sequence[PackedBatch], lr: Optional[float] = None,
                       noise: Optional[Sequence[torch.Tensor]] = None):
        """Same step for batches that already live on the device; returns device scalars."""
        ce_norm, gen_norm = self._normalisers(batches)
        # plain dense engine: the first micro-batch stores the layers' weight gradients, so they are not cleared
        store_first = (getattr(self, "store_first_enabled", True) and self.engine is not None
                       and type(self.engine).__name__ == "MoTEngine" and self.wp is None
                       and getattr(self.engine, "cp", None) is None and getattr(self.engine, "tp", None) is None
                       and not self.optim.cfg.frozen and not self.store.cfg.is_moe
                       and type(self.store).__name__ == "ParamStore")
        self.store.zero_grads(keep_layer_matrices=True) if store_first else self.store.zero_grads()
        acc = None
        if self.wp is not None:
            self.wp.begin_step()
            self.wp.single_micro = len(batches) == 1
        for i, b in enumerate(batches):
            self._last_micro = i == len(batches) - 1
            if self.wp is not None:
                self.wp.micro = i
            elif self._last_micro and hasattr(self.optim, "begin_step"):
                self.optim.begin_step()
            if self.engine is not None:
                self.engine.store_first = (store_first and i == 0) or (self.wp is not None and self.wp.store_layers)
                out = self.engine.forward_backward(b, noise[i] if noise else None, ce_norm, gen_norm)
                self.engine.store_first = False
            else:
                out = self._oracle_step(b, noise[i] if noise else None, ce_norm, gen_norm)
            acc = out if acc is None else {k: acc[k] + out[k] for k in acc}
        if self.optim.cfg.frozen:
            for a in self.store.sizes:
                if a != "mat" or self.engine is None:      # matrix buckets were cleared as they became ready
                    self._clear_frozen(a, 0, self.store.sizes[a])
        self.sync_tp_replicated_grads()
        if getattr(self.engine, "sel_bias", None):
            self.engine.update_selection_bias(self.dp_group)
        if self.profile_events is not None:      # [(start, end)] CUDA events around the optimizer step
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            self.optim.step(lr)
            e1.record()
            self.profile_events.append((e0, e1))
        else:
            self.optim.step(lr)
        if self.ema is not None:
            self._ema_update()
        self.step_idx += 1
        norm = getattr(self.optim, "last_grad_norm", None)
        if norm is not None and acc is not None:
            acc["grad_norm"] = norm.reshape(()) if norm.numel() == 1 else norm.sum()      # norm before clipping
        return acc

    def sync_tp_replicated_grads(self) -> None:
        """Tensor parallel: tensors that every rank of the group holds in full (embedding, heads, pixel front-ends,
        gains) see the same activations on every rank, but some of their gradients are summed with atomics, whose
        order differs from GPU to GPU; averaging them over the group before the update keeps the copies bit-identical
        for the whole run (the reference broadcasts / checks replicas instead: utils/parallel.py:112-243)."""
        tp = getattr(self.engine, "tp", None) if self.engine is not None else None
        if tp is None:
            return
        g = self.store.grad_arena
        for name, lo, hi in self.store.buckets("mat"):
            if name.startswith("layer."):
                continue                       # decoder matrices are sharded, not replicated
            step = tp.max_numel
            for a in range(lo, hi, step):
                b = min(hi, a + step)
                n = (b - a) // (8 * tp.world) * (8 * tp.world)
                if n:
                    tp.all_reduce_(g["mat"][a:a + n])
                if a + n < b:                  # a tail shorter than the all-reduce granule
                    dist.all_reduce(g["mat"][a + n:b], group=tp.group)
            g["mat"][lo:hi].mul_(1.0 / tp.world)
        dist.all_reduce(g["vec"], group=tp.group)
        g["vec"].mul_(1.0 / tp.world)

    # engine callbacks: overlap gradient reduce-scatter with the rest of backward, and the
    # weight all-gather of the previous step with this step's forward
    def _clear_frozen(self, arena: str, lo: int, hi: int) -> None:
        """Gradients of frozen ranges inside [lo, hi) are dropped (they must not reach the clipping norm)."""
        for s, e in (self.optim.cfg.frozen or {}).get(arena) or []:
            a, b = max(s, lo), min(e, hi)
            if b > a:
                self.store.grad_arena[arena][a:b].zero_()

    def _wp_layer_backward(self, l: int) -> None:
        self.wp.acquire_layer(l, l - 1)
        self.wp.begin_layer_backward(l)

    def _grads_ready(self, bucket: str) -> None:
        if self.wp is not None:          # reduce-scattered after every micro-batch: the staging slots are reused
            self.wp.reduce_bucket("mat", bucket)
            return
        if self._last_micro:
            if self.optim.cfg.frozen:
                for name, lo, hi in self.store.buckets("mat"):
                    if name == bucket:
                        self._clear_frozen("mat", lo, hi)
            self.optim.reduce_bucket("mat", bucket)

    def _weights_needed(self, bucket: str) -> None:
        if self.wp is not None:
            if bucket == "front":
                self.wp.acquire_resident()
            elif bucket.startswith("layer."):
                l = int(bucket.split(".")[1])
                self.wp.acquire_layer(l, l + 1)
            return
        if bucket == "front":
            self.optim.wait_bucket("vec", "vec")
        self.optim.wait_bucket("mat", bucket)

    def _oracle_step(self, b, noise, ce_norm, gen_norm):
        from ..models import oracle
        p = {k: v.detach().requires_grad_(True) for k, v in self.store.p.items()}
        if noise is None and b.gen_rows.numel():
            g = torch.Generator().manual_seed(int(b.noise_seed))
            noise = torch.randn(b.gen_x16.shape, generator=g)
        loss, parts = oracle.training_loss(p, b, self.cfg, noise, ce_norm, gen_norm)
        loss.backward()
        for k, v in p.items():
            if v.grad is not None:
                self.store.g[k].add_(v.grad.to(self.store.g[k].dtype))
        out = {"loss": loss.detach()}
        out.update({k: v for k, v in parts.items()})
        return out

    def _ema_update(self):
        for a, lst in self.optim.pieces.items():
            if self.wp is not None and a == "mat":
                from ..ops import fused
                n = self.ema[a].numel()               # shard and state share their offsets
                if self.store.shard.tensor.numel() < n or self.optim.state[a]["lo"].numel() < n:
                    raise ValueError("EMA shadow, weight shard and optimizer state disagree in size")   # before any launch
                fused.ema(self.ema[a], self.store.shard.tensor[:n], self.optim.state[a]["lo"][:n], self.ema_decay)
                continue
            if self.dev.type == "cuda":
                from ..ops import fused
                for _, _, _, mlo, mhi, so in lst:
                    n = mhi - mlo
                    fused.ema(self.ema[a][so:so + n], self.store.arena[a][mlo:mhi],
                              self.optim.state[a]["lo"][so:so + n], self.ema_decay)
            else:
                self.ema[a].mul_(self.ema_decay).add_(self.optim.state[a]["master"], alpha=1 - self.ema_decay)
