"""Pipeline parallelism: 1F1B schedule over NCCL / gloo point-to-point.

Reference: PipelineScheduler._forward_backward_step (training/sensenovalm/core/scheduler/
pipeline_scheduler.py:588-869), p2p helpers (core/scheduler/comm/p2p.py:123-264) and the shape /
dtype handshake (core/scheduler/comm/utils.py:66-137).  Differences: activations travel as one
contiguous tensor whose shape is agreed once per run (not per step), sends are asynchronous and are
only waited on when their buffer is reused, so they overlap the next micro-batch's compute, and the
schedule is a plain list of (op, micro-batch) pairs that a test can inspect.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def one_f_one_b(pp_size: int, pp_rank: int, num_micro: int) -> List[Tuple[str, int]]:
    """Order of forward ('F') and backward ('B') passes of one stage: ``pp_size - pp_rank - 1`` warm-up
    forwards, then alternating forward / backward, then the remaining backwards."""
    warm = min(pp_size - pp_rank - 1, num_micro)
    out: List[Tuple[str, int]] = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < num_micro:
        out.append(("F", f)); f += 1
        out.append(("B", b)); b += 1
    while b < num_micro:
        out.append(("B", b)); b += 1
    return out


def zero_bubble_h1(pp_size: int, pp_rank: int, num_micro: int) -> List[Tuple[str, int]]:
    """ZB-H1 order of one stage: the backward pass is split into 'B' (gradient with respect to the
    stage input, which the previous stage is waiting for) and 'W' (weight gradients, which nobody
    waits for).  Same warm-up and same activation memory as 1F1B; every 'W' is delayed into the slot
    where 1F1B would idle, so the cool-down bubble of stage r shrinks by the time of r weight-gradient
    passes.  Reference: ZeroBubblePipelineScheduler with its WeightGradStore
    (training/sensenovalm/core/scheduler/pipeline_scheduler.py:122-166, :929-1180)."""
    warm = min(pp_size - pp_rank - 1, num_micro)
    out: List[Tuple[str, int]] = [("F", i) for i in range(warm)]
    f, b, w = warm, 0, 0
    defer = pp_rank                      # weight-gradient passes this stage may hold back
    while f < num_micro:
        out.append(("F", f)); f += 1
        out.append(("B", b)); b += 1
        if b - w > defer:
            out.append(("W", w)); w += 1
    while b < num_micro:
        out.append(("B", b)); b += 1
        if b - w > defer or b == num_micro:
            out.append(("W", w)); w += 1
    while w < num_micro:
        out.append(("W", w)); w += 1
    return out


def partition_uniform(num_layers: int, pp_size: int) -> List[Tuple[int, int]]:
    """Layer ranges per stage, remainder spread over the last stages (core/parallel/shard.py:181-207)."""
    base, rem = divmod(num_layers, pp_size)
    out, s = [], 0
    for r in range(pp_size):
        n = base + (1 if r >= pp_size - rem else 0)
        out.append((s, s + n)); s += n
    return out


@dataclass
class _Meta:
    shape: Tuple[int, ...]
    dtype: torch.dtype


_DT = [torch.float32, torch.bfloat16, torch.float16, torch.int64, torch.int32]


def send_meta(t: torch.Tensor, dst: int, group=None):
    info = torch.tensor([t.dim(), _DT.index(t.dtype)] + list(t.shape) + [0] * (8 - t.dim()), dtype=torch.int64,
                        device=t.device if t.is_cuda else "cpu")
    dist.send(info, dst, group=group)


def recv_meta(src: int, device, group=None) -> _Meta:
    info = torch.zeros(10, dtype=torch.int64, device=device)
    dist.recv(info, src, group=group)
    v = info.tolist()
    return _Meta(tuple(v[2:2 + v[0]]), _DT[v[1]])


def make_pipeline_groups(ranks: Sequence[int], backend: Optional[str] = None):
    """Two process groups over the pipeline's ranks: one carries activations downstream, the other carries
    gradients upstream.  Every rank of the job must call this (``dist.new_group`` is collective)."""
    return dist.new_group(list(ranks), backend=backend), dist.new_group(list(ranks), backend=backend)


class PipelineStage:
    """Runs one stage of a 1F1B or ZB-H1 pipeline.

    ``forward_fn(x_in or None, micro_index) -> tensor``: the stage's computation; on the last stage it
    returns the scalar loss of the micro-batch.  By default the backward pass is autograd's.  An engine
    with an explicit backward passes ``backward_fn(micro_index, grad_out or None) -> grad_in or None``
    (and, for the zero-bubble schedule, ``wgrad_fn(micro_index)``); then no autograd graph is used.

    Communication.  Activations (stage r -> r+1) and gradients (r+1 -> r) travel on two different
    process groups, i.e. two communicators with a stream each.  Within one direction both ends issue
    their transfers in micro-batch order, so each communicator sees a matching FIFO sequence on both
    sides; a send of one direction can never queue in front of a receive of the other direction, which
    is the circular wait that separate ``isend`` / ``recv`` calls on ONE communicator produce once a
    message is larger than the eager buffer (the reference avoids the same cycle with fused
    ``batch_isend_irecv`` pairs, core/scheduler/comm/p2p.py:123-264).  The host never blocks on a
    transfer: receives are posted one schedule slot ahead and only the consuming stream waits, so the
    copy of micro-batch i+1 overlaps the compute of micro-batch i.  With the NCCL backend a single shared
    group is refused.
    """

    def __init__(self, forward_fn: Callable, pp_rank: int, pp_size: int, prev_rank: Optional[int],
                 next_rank: Optional[int], device="cpu", group=None, schedule: str = "1f1b",
                 params: Optional[Sequence[torch.Tensor]] = None, bwd_group=None,
                 backward_fn: Optional[Callable] = None, wgrad_fn: Optional[Callable] = None):
        """``schedule``: "1f1b" or "zero_bubble" (needs ``params``: the stage's parameters, whose
        gradients are then computed in separate, deferred 'W' passes; or ``wgrad_fn``).
        ``group`` carries activations, ``bwd_group`` gradients (see :func:`make_pipeline_groups`)."""
        if schedule not in ("1f1b", "zero_bubble"):
            raise ValueError(f"unknown pipeline schedule {schedule!r}")
        if schedule == "zero_bubble" and params is None and wgrad_fn is None:
            raise ValueError("the zero-bubble schedule needs the stage's parameter list or a wgrad_fn")
        self.schedule, self.params = schedule, list(params) if params is not None else None
        self.fn, self.bwd_fn, self.wgrad_fn = forward_fn, backward_fn, wgrad_fn
        self.rank, self.size = pp_rank, pp_size
        self.prev, self.next, self.dev = prev_rank, next_rank, torch.device(device)
        self.group, self.bwd_group = group, bwd_group if bwd_group is not None else group
        if pp_size > 1 and dist.is_initialized() and dist.get_backend(group) == "nccl" and self.bwd_group is group:
            raise ValueError("with the NCCL backend activations and gradients need a communicator each: pass "
                             "group=, bwd_group= from make_pipeline_groups(); one shared communicator can "
                             "deadlock on messages larger than its eager buffer")
        self.meta_in: Optional[_Meta] = None
        self.meta_out: Optional[_Meta] = None
        self._meta_sent = False
        self._pending: List = []
        self._posted = {}          # (op, micro-batch) -> (buffer, work) of a receive already posted
        self.trace: List[Tuple[str, int]] = []

    @property
    def first(self):
        return self.rank == 0

    @property
    def last(self):
        return self.rank == self.size - 1

    # -- receives: posted ahead, waited on by the consumer ----------------------------------------
    def _needs_recv(self, op: str) -> bool:
        return (op == "F" and not self.first) or (op == "B" and not self.last)

    def _post(self, op: str, i: int) -> None:
        if (op, i) in self._posted or not self._needs_recv(op):
            return
        if op == "F":
            if self.meta_in is None:
                self.meta_in = recv_meta(self.prev, self.dev if self.dev.type == "cuda" else "cpu", self.group)
            t = torch.empty(self.meta_in.shape, dtype=self.meta_in.dtype, device=self.dev)
            self._posted[(op, i)] = (t, dist.irecv(t, self.prev, group=self.group))
        else:
            if self.meta_out is None:
                return             # the output shape is known after this stage's first forward
            t = torch.empty(self.meta_out.shape, dtype=self.meta_out.dtype, device=self.dev)
            self._posted[(op, i)] = (t, dist.irecv(t, self.next, group=self.bwd_group))

    def _take(self, op: str, i: int) -> torch.Tensor:
        self._post(op, i)
        t, w = self._posted.pop((op, i))
        w.wait()
        return t

    def _isend(self, t, dst, group):
        self._pending = [w for w in self._pending if not w.is_completed()]
        self._pending.append(dist.isend(t.contiguous(), dst, group=group))

    def run(self, num_micro: int) -> List[torch.Tensor]:
        """Executes the schedule; returns the micro-batch losses (last stage) or []."""
        inputs, outputs, losses = {}, {}, []
        wstore = {}      # micro-batch -> (output, upstream gradient): the deferred weight-gradient work
        zb = self.schedule == "zero_bubble"
        order = zero_bubble_h1(self.size, self.rank, num_micro) if zb else one_f_one_b(self.size, self.rank, num_micro)
        comm_ops = [(op, i) for op, i in order if self._needs_recv(op)]
        nxt = {c: comm_ops[k + 1] for k, c in enumerate(comm_ops[:-1])}
        for op, i in order:
            self.trace.append((op, i))
            if op == "W":
                if self.wgrad_fn is not None:
                    self.wgrad_fn(i)
                    continue
                y, g = wstore.pop(i)
                ps = [p for p in self.params if p.requires_grad]
                grads = torch.autograd.grad(y, ps, g, allow_unused=True)
                for p, gr in zip(ps, grads):
                    if gr is not None:
                        p.grad = gr if p.grad is None else p.grad + gr
                continue
            self._post(op, i)
            if (op, i) in nxt:
                self._post(*nxt[(op, i)])      # the next transfer flows in while this pass computes
            if op == "F":
                x = None
                if not self.first:
                    x = self._take("F", i)
                    if self.bwd_fn is None:
                        x.requires_grad_(True)
                y = self.fn(x, i)
                inputs[i], outputs[i] = x, y
                if self.last:
                    losses.append(y.detach())
                else:
                    if not self._meta_sent:
                        send_meta(y, self.next, self.group)
                        self._meta_sent = True
                        self.meta_out = _Meta(tuple(y.shape), y.dtype)
                    self._isend(y.detach(), self.next, self.group)
            else:
                y, x = outputs.pop(i), inputs.pop(i)
                g = None if self.last else self._take("B", i)
                if self.bwd_fn is not None:
                    gx = self.bwd_fn(i, g)
                    if not self.first:
                        self._isend(gx, self.prev, self.bwd_group)
                elif zb:
                    # input gradient now (the previous stage waits for it), weight gradients later
                    if not self.first:
                        gx, = torch.autograd.grad(y, [x], g, retain_graph=True)
                        self._isend(gx, self.prev, self.bwd_group)
                    wstore[i] = (y, g)
                else:
                    if self.last:
                        y.backward()
                    else:
                        y.backward(g)
                    if not self.first:
                        self._isend(x.grad, self.prev, self.bwd_group)
        for w in self._pending:
            w.wait()
        self._pending.clear()
        return losses


def allreduce_shared_grads(params: Sequence[torch.Tensor], group=None) -> None:
    """Sums the gradients of parameters that live on both pipeline ends (tied embedding / head:
    core/gradient_handler.py:37-78)."""
    for p in params:
        if p.grad is not None:
            dist.all_reduce(p.grad, group=group)
