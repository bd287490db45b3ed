"""Weight-parallel training ("ISP" weight parallel of the reference, its shipped 8B mode: ``wp=8, tp=1``).

Reference mechanism (training/sensenovalm/core/parallel/comm/isp.py:312-850,
training/sensenovalm/model/modules/linear.py:169-295): every linear holds 1/wp of its weight; the
weight is all-gathered before the forward GEMM (prefetched one block ahead), again before the
recompute / backward GEMMs, and the weight gradient is reduce-scattered to the owning shard; the
optimizer (ZeRO-1 inside the weight-parallel group) only ever sees the shard.

Here the same contract is kept at the granularity the engine already communicates in, the
*bucket* (``front``, one per decoder layer, ``head``):

* at rest a rank holds piece ``r`` of every bucket: ``shard`` (bf16 weights, symmetric memory so that
  peers can read it), ``gshard`` (reduced gradients) and the optimizer state of the piece;
* a decoder layer's weights exist in full only inside a ring of ``ring`` gathered buffers: layer
  ``l`` is assembled in slot ``l % ring`` by ``wp_gather`` (this package's peer-load kernel, csrc/optim.cu)
  on a side stream while layer ``l-1`` (forward) or ``l+1`` (backward) computes; the backward pass
  starts on the slot the forward pass left behind, so a step gathers every layer twice;
* weight gradients of a layer are accumulated by the GEMM epilogues in a full-size staging slot
  (ring of two, symmetric memory); when the layer's backward is done the rank signals its peers,
  and ``rs_pull`` sums piece ``r`` of all ranks' staging slots into ``gshard`` on another side
  stream (reduce-scatter + cast + squared norm in one pass) while the next layer's backward runs;
* the small ``front`` / ``head`` buckets (embedding, pixel front-ends, heads) are gathered once per
  step into resident buffers; the ``vec`` arena (gains, biases) stays replicated.

Flag words in symmetric memory order everything across GPUs (release / acquire at system scope,
bounded waits): *weights ready* (after the optimizer step, before the first gather of the next step),
*gradients ready* (per bucket) and *pulled* (per bucket: the staging slot may be reused).
"""
from __future__ import annotations

import os

import ctypes
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..config import ModelConfig
from ..models.params import ALIGN, ParamStore, build_specs
from ..train.optimizer import AdamConfig, ZeroAdamW


def _round_up(n, a):
    return (n + a - 1) // a * a


class _LocalPeers:
    """Stand-in for a SymmetricBuffer when the group has one rank (tests on one GPU)."""

    def __init__(self, numel, dtype, device):
        self.tensor = torch.zeros(numel, dtype=dtype, device=device)
        self.world, self.rank = 1, 0
        self.ptrs = [self.tensor.data_ptr()]
        self.c_ptrs = (ctypes.c_longlong * 1)(*self.ptrs)

    def barrier(self):
        pass


def _symmetric(numel, dtype, device, group, world):
    if world == 1:
        return _LocalPeers(numel, dtype, device)
    from .symm import SymmetricBuffer
    return SymmetricBuffer(numel, dtype, device, group)


class WeightParallelStore:
    """Parameter storage of the weight-parallel mode.  Presents the attributes of :class:`ParamStore` that the
    engine, the trainer and the optimizer use (``p``, ``g``, ``arena``, ``grad_arena``, ``sizes``, ``buckets`` ...),
    with the matrix arena replaced by shard + gathered buffers."""

    def __init__(self, cfg: ModelConfig, device, group=None, dtype=torch.bfloat16, ring: int = 2):
        if cfg.is_moe and cfg.ep_size > 1:
            raise NotImplementedError("weight parallel covers the dense arenas; expert-parallel experts stay rank-local")
        if ring < 2:
            raise ValueError("the gathered-weight ring needs at least two slots (one computing, one arriving)")
        self.cfg, self.device, self.dtype, self.group, self.ring = cfg, torch.device(device), dtype, group, ring
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.ep_rank = 0
        self.symm = None
        self.specs = build_specs(cfg)
        self.by_name = {s.name: s for s in self.specs}
        layout = ParamStore.__new__(ParamStore)             # offsets / sizes / buckets exactly as the full store
        layout.cfg, layout.specs = cfg, self.specs
        self.offsets: Dict[str, Tuple[str, int]] = {}
        sizes = {"mat": 0, "vec": 0}
        for s in self.specs:
            if s.arena == "exp":
                raise NotImplementedError("expert arenas are not weight parallel")
            self.offsets[s.name] = (s.arena, sizes[s.arena])
            sizes[s.arena] += _round_up(s.numel, ALIGN)
        mult = 8 * ALIGN * self.world
        self.sizes = {k: _round_up(max(v, ALIGN), mult) for k, v in sizes.items()}
        layout.offsets, layout.sizes = self.offsets, self.sizes
        self._layout = layout
        W = self.world
        # pieces of the matrix arena: bucket -> (lo, hi, per, shard offset)
        self.mat_buckets: List[Tuple[str, int, int]] = layout.buckets("mat")
        self.piece: Dict[str, Tuple[int, int, int, int]] = {}
        off = 0
        for name, lo, hi in self.mat_buckets:
            if (hi - lo) % (W * 8):
                raise ValueError(f"bucket {name} ({hi - lo} elements) does not split over {W} ranks")
            per = (hi - lo) // W
            self.piece[name] = (lo, hi, per, off)
            off += per
        self.shard_numel = off
        layer_sizes = {hi - lo for n, lo, hi in self.mat_buckets if n.startswith("layer.")}
        if len(layer_sizes) > 1:
            raise ValueError("decoder-layer buckets differ in size; the gathered-weight ring needs one size")
        self.layer_numel = layer_sizes.pop() if layer_sizes else 0
        dev = self.device
        self.shard = _symmetric(self.shard_numel, dtype, dev, group, W)
        self.gshard = torch.zeros(self.shard_numel, dtype=dtype, device=dev)
        self.wres: Dict[str, torch.Tensor] = {}
        self.gres = {}
        for name, lo, hi in self.mat_buckets:
            if not name.startswith("layer."):
                self.wres[name] = torch.zeros(hi - lo, dtype=dtype, device=dev)
                self.gres[name] = _symmetric(hi - lo, dtype, dev, group, W)
        self.wring = [torch.zeros(self.layer_numel, dtype=dtype, device=dev) for _ in range(ring)] if self.layer_numel else []
        self.gring = [_symmetric(self.layer_numel, dtype, dev, group, W) for _ in range(2)] if self.layer_numel else []
        self.arena = {"vec": torch.zeros(self.sizes["vec"], dtype=dtype, device=dev)}
        self.grad_arena = {"vec": torch.zeros(self.sizes["vec"], dtype=torch.float32, device=dev)}
        self.p: Dict[str, torch.Tensor] = {}
        self.g: Dict[str, torch.Tensor] = {}
        bounds = [(name, lo, hi) for name, lo, hi in self.mat_buckets]
        for s in self.specs:
            a, o = self.offsets[s.name]
            if a == "vec":
                self.p[s.name] = self.arena["vec"][o:o + s.numel].view(s.shape)
                self.g[s.name] = self.grad_arena["vec"][o:o + s.numel].view(s.shape)
                continue
            b = next(n for n, lo, hi in bounds if lo <= o < hi)
            rel = o - self.piece[b][0]
            if b.startswith("layer."):
                l = int(b.split(".")[1])
                wbuf, gbuf = self.wring[l % ring], self.gring[l % 2].tensor
            else:
                wbuf, gbuf = self.wres[b], self.gres[b].tensor
            self.p[s.name] = wbuf[rel:rel + s.numel].view(s.shape)
            self.g[s.name] = gbuf[rel:rel + s.numel].view(s.shape)

    # ---- the ParamStore surface -------------------------------------------------------------------------
    def buckets(self, arena: str):
        return self._layout.buckets(arena)

    def segments(self, arena: str):
        return ParamStore.segments(self._layout, arena)

    def named_parameters(self):
        raise NotImplementedError("weight-parallel weights are sharded: use to_param_store() for full tensors")

    def zero_grads(self) -> None:
        """Clears the reduced gradients, the resident staging buffers and the vec gradients; a decoder layer's
        staging slot is cleared right before that layer's backward (WeightParallelAdamW.begin_layer_backward)."""
        self.gshard.zero_()
        self.grad_arena["vec"].zero_()
        for sb in self.gres.values():
            sb.tensor.zero_()

    def bucket_of_layer(self, l: int) -> str:
        return f"layer.{l}"

    def my_piece(self, name: str) -> torch.Tensor:
        _, _, per, so = self.piece[name]
        return self.shard.tensor[so:so + per]

    # ---- initialisation / conversion ---------------------------------------------------------------------
    def _scatter_into_shard(self, arena_off: int, values: torch.Tensor) -> None:
        """Writes ``values`` (the arena elements [arena_off, arena_off + n)) into the shard where they fall into
        one of this rank's pieces."""
        n = values.numel()
        for name, (lo, hi, per, so) in self.piece.items():
            mlo = lo + self.rank * per
            a, b = max(arena_off, mlo), min(arena_off + n, mlo + per)
            if b > a:
                self.shard.tensor[so + (a - mlo):so + (b - mlo)].copy_(values[a - arena_off:b - arena_off])

    def init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        """The same random stream as ``ParamStore.init_weights`` (every rank draws all of it and keeps its pieces), so
        that a weight-parallel run starts from exactly the weights of a data-parallel run with that seed."""
        g = torch.Generator(device=self.device).manual_seed(seed)
        torch.Generator(device=self.device).manual_seed(seed + 7919)          # the full store's expert generator (unused)
        L = max(1, self.cfg.num_layers)
        for s in self.specs:
            a, o = self.offsets[s.name]
            if s.init in ("ones", "zeros"):
                if a == "vec":
                    self.p[s.name].fill_(1.0 if s.init == "ones" else 0.0)
                else:
                    self._scatter_into_shard(o, torch.full((s.numel,), 1.0 if s.init == "ones" else 0.0,
                                                           dtype=self.dtype, device=self.device))
                continue
            sd = std / (2 * L) ** 0.5 if s.init == "out_normal" else std
            step = 1 << 26
            for i in range(0, s.numel, step):
                n = min(step, s.numel - i)
                chunk = (torch.randn(n, device=self.device, generator=g) * sd).to(self.dtype)
                if a == "vec":
                    self.p[s.name].view(-1)[i:i + n] = chunk
                else:
                    self._scatter_into_shard(o + i, chunk)

    def load_from(self, full: ParamStore) -> None:
        """Takes this rank's pieces (and the whole vec arena) from a full store."""
        self.arena["vec"].copy_(full.arena["vec"][: self.sizes["vec"]].to(self.dtype))
        for name, (lo, hi, per, so) in self.piece.items():
            mlo = lo + self.rank * per
            self.shard.tensor[so:so + per].copy_(full.arena["mat"][mlo:mlo + per].to(self.dtype))

    def to_param_store(self, device=None) -> ParamStore:
        """A full :class:`ParamStore` (weights only) assembled from all ranks' shards: checkpoints and exports go
        through it.  Collective over the group."""
        full = ParamStore(self.cfg, device=device or self.device, dtype=self.dtype, with_grads=False,
                          shard_multiple=8 * ALIGN * self.world)
        full.arena["vec"].copy_(self.arena["vec"])
        for name, (lo, hi, per, so) in self.piece.items():
            mine = self.shard.tensor[so:so + per]
            if self.world == 1:
                full.arena["mat"][lo:hi].copy_(mine)
            else:
                tmp = torch.empty(hi - lo, dtype=self.dtype, device=self.device)
                dist.all_gather_into_tensor(tmp, mine.contiguous(), group=self.group)
                full.arena["mat"][lo:hi].copy_(tmp)
        return full


class WeightParallelAdamW(ZeroAdamW):
    """Gather / reduce-scatter schedule and the ZeRO-1 update of the weight-parallel mode (see the module text)."""

    def __init__(self, store: WeightParallelStore, cfg: AdamConfig, group=None, grad_divisor: float = 1.0,
                 gather_grid: int = 96, pull_grid: int = 296):
        if store.device.type != "cuda":
            raise ValueError("the weight-parallel engine runs on CUDA devices")
        if cfg.frozen:
            raise NotImplementedError("frozen parameter ranges are not supported in weight-parallel mode")
        self.wp = store
        super().__init__(store, cfg, group=group, grad_divisor=grad_divisor)
        W = self.world
        # CTAs of the side-stream kernels (they share the SMs with the GEMMs they run beside); environment overrides
        # for tuning runs
        self.gather_grid = int(os.environ.get("SNU1_WP_GATHER_GRID", gather_grid))
        self.pull_grid = int(os.environ.get("SNU1_WP_PULL_GRID", pull_grid))
        names = [n for n, _, _ in store.mat_buckets]
        self.slot = {n: (3 * i, 3 * i + 1) for i, n in enumerate(names)}       # (gradients ready, pulled)
        self.slot_w = 3 * len(names)                                            # weights ready (one for all buckets)
        self.flags = _symmetric((3 * len(names) + 1) * W, torch.int32, self.dev, group, W)
        self.side_ag = torch.cuda.Stream(device=self.dev)
        self.side_rs = torch.cuda.Stream(device=self.dev)
        self.seq = 0                       # one per micro-batch backward: value of the gradient / pulled flags
        self.micro = 0
        self.slot_content = [-1] * store.ring
        self.gather_ev: Dict[int, torch.cuda.Event] = {}
        self.resident_ready = False
        self.gring_owner = [None, None]    # (layer, seq) whose gradients sit in the staging slot
        # the engine stores (does not add) a decoder layer's four weight gradients into its staging slot, and the
        # slot holds nothing else, so it needs no clearing between uses
        self.store_layers = True
        self._weights_flag_waited = -1
        self.gathers = 0
        self.flags.barrier()

    # the vec arena keeps the plain ZeRO layout of the base class; the matrix arena is addressed through the shard
    def _call(self, name, *args):
        from ..ops import _lib
        _lib.call(name, *args)

    def _wait_flag(self, slot, value, stream):
        from ..ops._lib import c_int, c_void_p
        if self.world > 1:
            self._call("wait_flags", c_void_p(self.flags.tensor.data_ptr()), c_int(self.world), c_int(slot),
                       c_int(value), c_void_p(stream.cuda_stream))

    def _signal(self, slot, value, stream):
        from ..ops._lib import c_int, c_void_p
        if self.world > 1:
            self._call("signal_peers", self.flags.c_ptrs, c_int(self.world), c_int(self.rank), c_int(slot),
                       c_int(value), c_void_p(stream.cuda_stream))

    # ---- weights: gather ------------------------------------------------------------------------------------
    def _gather(self, bucket: str, dst: torch.Tensor, stream) -> None:
        from ..ops._lib import c_int, c_ll, c_void_p
        lo, hi, per, so = self.wp.piece[bucket]
        if self._weights_flag_waited != self.step_count:
            # the first gather after an optimizer step: every rank's shard must hold that step's weights
            self._wait_flag(self.slot_w, self.step_count, stream)
            self._weights_flag_waited = self.step_count
        self._call("wp_gather", self.wp.shard.c_ptrs, c_int(self.world), c_ll(so), c_ll(per),
                   c_void_p(dst.data_ptr()), c_int(self.gather_grid), c_void_p(stream.cuda_stream))
        self.gathers += 1

    def _issue_layer_gather(self, l: int) -> None:
        slot = l % self.wp.ring
        cur = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(cur)                      # everything that still reads the slot's old content is queued before this
        self.side_ag.wait_event(ev)
        self._gather(f"layer.{l}", self.wp.wring[slot], self.side_ag)
        done = torch.cuda.Event()
        done.record(self.side_ag)
        self.gather_ev[l] = done
        self.slot_content[slot] = l

    def acquire_layer(self, l: int, next_l: Optional[int]) -> None:
        """Makes layer ``l``'s full weights valid in its ring slot for the kernels queued after this call and starts
        the gather of ``next_l`` (the layer the pass visits next) behind them."""
        slot = l % self.wp.ring
        if self.slot_content[slot] != l:
            self._issue_layer_gather(l)
        ev = self.gather_ev.get(l)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        if next_l is not None and 0 <= next_l < self.wp.cfg.num_layers and \
                self.slot_content[next_l % self.wp.ring] != next_l:
            self._issue_layer_gather(next_l)

    def acquire_resident(self) -> None:
        """``front`` and ``head`` buckets: gathered once per step."""
        if self.resident_ready:
            return
        cur = torch.cuda.current_stream()
        for name, buf in self.wp.wres.items():
            self._gather(name, buf, cur)
        self.resident_ready = True

    # ---- gradients: staging slots and reduce-scatter -----------------------------------------------------------
    def begin_step(self):
        self.norm_sq.zero_()
        self.micro = 0

    def begin_micro_backward(self):
        """Start of the backward pass of one micro-batch.  From the second micro-batch on, the resident staging
        buffers (front / head) still hold the previous micro-batch's gradients, already pulled into ``gshard``:
        once every peer has pulled them they are cleared (a decoder layer's slot is cleared per layer)."""
        self.seq += 1
        if self.micro > 0:
            cur = torch.cuda.current_stream()
            cur.wait_stream(self.side_rs)
            for name, sb in self.wp.gres.items():
                self._wait_flag(self.slot[name][1], self.seq - 1, cur)
                sb.tensor.zero_()

    def begin_layer_backward(self, l: int) -> None:
        """Before the backward of layer ``l`` writes its staging slot: the peers must have pulled the gradients of
        the layer that used the slot before (the slot is then overwritten by stores, or cleared first when
        ``store_layers`` is off)."""
        k = l % 2
        owner = self.gring_owner[k]
        cur = torch.cuda.current_stream()
        if owner is not None:
            if self.world == 1:
                cur.wait_stream(self.side_rs)       # no flags with one rank: order behind the own pull
            self._wait_flag(self.slot[f"layer.{owner[0]}"][1], owner[1], cur)
        if not self.store_layers:
            self.wp.gring[k].tensor.zero_()
        self.gring_owner[k] = (l, self.seq)

    def reduce_bucket(self, arena: str, name: str) -> None:
        from ..ops._lib import c_int, c_ll, c_void_p
        if arena != "mat":
            return
        cur = torch.cuda.current_stream()
        slot_g, slot_p = self.slot[name]
        self._signal(slot_g, self.seq, cur)
        self.side_rs.wait_stream(cur)
        self._wait_flag(slot_g, self.seq, self.side_rs)
        lo, hi, per, so = self.wp.piece[name]
        if name.startswith("layer."):
            src = self.wp.gring[int(name.split(".")[1]) % 2]
        else:
            src = self.wp.gres[name]
        in_kernel_norm = self.single_micro
        self._call("rs_pull", src.c_ptrs, c_int(self.world), c_ll(self.rank * per), c_ll(per),
                   c_void_p(self.wp.gshard[so:so + per].data_ptr()), c_int(1 if self.micro > 0 else 0),
                   c_void_p(self.norm_sq.data_ptr() if in_kernel_norm else None), c_int(self.pull_grid),
                   c_void_p(self.side_rs.cuda_stream))
        self._signal(slot_p, self.seq, self.side_rs)

    single_micro = True

    def end_micro(self):
        self.micro += 1

    # ---- the step ------------------------------------------------------------------------------------------------
    def step(self, lr: Optional[float] = None) -> None:
        from ..ops import fused
        c = self.cfg
        lr = self.lr if lr is None else lr
        cur = torch.cuda.current_stream()
        cur.wait_stream(self.side_rs)
        self.step_count += 1
        if not self.single_micro:
            fused.sumsq(self.wp.gshard, self.norm_sq)
        # vec arena: replicated weights, gradients summed with NCCL, this rank's piece contributes to the norm
        if self.world > 1:
            dist.all_reduce(self.store.grad_arena["vec"], group=self.group)
        for _, _, _, mlo, mhi, _ in self.pieces["vec"]:
            fused.sumsq(self.store.grad_arena["vec"][mlo:mhi], self.norm_sq)
        if self.world > 1:
            dist.all_reduce(self.norm_sq, op=dist.ReduceOp.SUM, group=self.group)
        nsq = self.norm_sq
        pre = 1.0 / self.grad_divisor
        self.last_grad_norm = nsq.detach().float().sqrt() * pre      # device scalar, logged by the trainer
        st = self.state["mat"]
        for s, e, sc, wd, so in self.own_ranges("mat"):
            n = e - s
            fused.adamw(self.wp.shard.tensor[so:so + n], st["lo"][so:so + n], self.wp.gshard[so:so + n],
                        st["m"][so:so + n], st["v"][so:so + n], lr=lr * sc, beta1=c.beta1, beta2=c.beta2, eps=c.eps,
                        weight_decay=wd, step=self.step_count, grad_prescale=pre, norm_sq=nsq,
                        max_norm=c.clip_grad_norm, skipped=self.skipped)
        st = self.state["vec"]
        P, G = self.store.arena["vec"], self.store.grad_arena["vec"]
        for s, e, sc, wd, so in self.own_ranges("vec"):
            n = e - s
            fused.adamw(P[s:e], st["lo"][so:so + n], G[s:e], st["m"][so:so + n], st["v"][so:so + n], lr=lr * sc,
                        beta1=c.beta1, beta2=c.beta2, eps=c.eps, weight_decay=wd, step=self.step_count,
                        grad_prescale=pre, norm_sq=nsq, max_norm=c.clip_grad_norm, skipped=self.skipped)
        if self.world > 1:
            for name, lo, hi, mlo, mhi, _ in self.pieces["vec"]:
                dist.all_gather_into_tensor(P[lo:hi], P[mlo:mhi], group=self.group)
        self._signal(self.slot_w, self.step_count, cur)
        # every gathered copy is stale now
        self.slot_content = [-1] * self.wp.ring
        self.gather_ev.clear()
        self.resident_ready = False
        # gathers of the next step run on side_ag: they must start after this step's update of the local shard
        self.side_ag.wait_stream(cur)

    def reduce_gradients(self):
        torch.cuda.current_stream().wait_stream(self.side_rs)

    def gather_params(self):
        return

    def wait_bucket(self, arena: str, name: str) -> None:
        return

    def wait_all(self) -> None:
        return
