"""Tensor / sequence / Ulysses parallel building blocks as autograd functions over a process group.

Reference: core/parallel/comm/utils.py:41-220 (gather / split / reduce autograd wrappers),
comm/tensor.py:94-217 (Megatron TP: all-reduce after the row-parallel product, and sequence
parallel: all-gather before the column-parallel product, reduce-scatter after the row-parallel
one), comm/isp.py:925-994 (``_SeqAllToAll``: scatter heads / gather sequence and back), and
ops/cross_entropy.py:159-280 (vocab-parallel cross entropy with three all-reduces).
These run on any backend (gloo in the CPU tests).  On B200 the row-parallel reduce-scatter and the
weight all-gather have fused kernels in ``parallel/fused_ops.py``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F


def _ws(group):
    return dist.get_world_size(group) if dist.is_initialized() else 1


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel linear)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel linear)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherSeq(torch.autograd.Function):
    """All-gather along dim 0 forward, reduce-scatter backward (sequence parallel input)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = _ws(group)
        out = torch.empty((x.shape[0] * w,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = _ws(ctx.group)
        out = torch.empty((g.shape[0] // w,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _ReduceScatterSeq(torch.autograd.Function):
    """Reduce-scatter along dim 0 forward, all-gather backward (sequence parallel output)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = _ws(group)
        out = torch.empty((x.shape[0] // w,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = _ws(ctx.group)
        out = torch.empty((g.shape[0] * w,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _SeqAllToAll(torch.autograd.Function):
    """Ulysses exchange.  x [S_local, heads, D] -> [S_local * w, heads / w, D] (scatter heads, gather
    sequence) when ``to_heads``; the inverse otherwise.  Backward is the inverse exchange."""

    @staticmethod
    def forward(ctx, x, group, to_heads):
        ctx.group, ctx.to_heads = group, to_heads
        return _a2a(x, group, to_heads)

    @staticmethod
    def backward(ctx, g):
        return _a2a(g, ctx.group, not ctx.to_heads), None, None


def _a2a(x, group, to_heads):
    w = _ws(group)
    if w == 1:
        return x
    S, Hh, D = x.shape
    if to_heads:
        # send head block j to rank j; receive everyone's sequence slice of my head block
        inp = x.reshape(S, w, Hh // w, D).permute(1, 0, 2, 3).contiguous()
        out = torch.empty_like(inp)
        dist.all_to_all_single(out, inp, group=group)
        return out.reshape(w * S, Hh // w, D)
    inp = x.reshape(w, S // w, Hh, D).contiguous()
    out = torch.empty_like(inp)
    dist.all_to_all_single(out, inp, group=group)
    return out.permute(1, 0, 2, 3).reshape(S // w, w * Hh, D)


copy_to_tp = lambda x, group=None: _CopyToTP.apply(x, group)
reduce_from_tp = lambda x, group=None: _ReduceFromTP.apply(x, group)
gather_seq = lambda x, group=None: _GatherSeq.apply(x, group)
reduce_scatter_seq = lambda x, group=None: _ReduceScatterSeq.apply(x, group)
seq_all_to_all = lambda x, group=None, to_heads=True: _SeqAllToAll.apply(x, group, to_heads)


def column_parallel_linear(x, w_shard, group=None, sequence_parallel=False):
    """``w_shard`` [N / tp, K].  With sequence parallel the input is sequence-split and gathered first."""
    x = gather_seq(x, group) if sequence_parallel else copy_to_tp(x, group)
    return F.linear(x, w_shard)


def row_parallel_linear(x, w_shard, group=None, sequence_parallel=False):
    """``w_shard`` [N, K / tp]; the partial products are summed (all-reduce) or reduce-scattered."""
    y = F.linear(x, w_shard)
    return reduce_scatter_seq(y, group) if sequence_parallel else reduce_from_tp(y, group)


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, group):
        w, r = _ws(group), (dist.get_rank(group) if dist.is_initialized() else 0)
        Vp = logits.shape[-1]
        lo = r * Vp
        lf = logits.float()
        mx = lf.max(dim=-1).values
        if w > 1:
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
        ex = (lf - mx[:, None]).exp()
        se = ex.sum(-1)
        inside = (target >= lo) & (target < lo + Vp)
        local_t = (target - lo).clamp(0, Vp - 1)
        tl = torch.where(inside, lf.gather(1, local_t[:, None])[:, 0] - mx, torch.zeros_like(mx))
        if w > 1:
            dist.all_reduce(se, group=group)
            dist.all_reduce(tl, group=group)
        loss = se.log() - tl
        ctx.save_for_backward(ex / se[:, None], inside, local_t)
        return loss

    @staticmethod
    def backward(ctx, g):
        p, inside, local_t = ctx.saved_tensors
        grad = p.clone()
        grad[torch.arange(p.shape[0], device=p.device)[inside], local_t[inside]] -= 1.0
        return grad * g[:, None], None, None


def vocab_parallel_cross_entropy(logits_shard, target, group=None):
    """Per-row CE when the vocabulary dimension of ``logits_shard`` [R, V / tp] is split over the group."""
    return _VocabParallelCE.apply(logits_shard, target, group)
