"""Capacity-based top-k gating (GShard style): the alternative to the dropless router.

Every expert accepts at most ``capacity = max(min_capacity, ceil(capacity_factor * k * S / E))``
token copies; copies are admitted choice by choice (all first choices in row order, then all second
choices, ...), later ones are dropped, and the surviving gate values of a token are renormalised.
The reference builds dense [S, E, C] one-hot dispatch / combine tensors and contracts them with
einsum (training/sensenovalm/model/moe/gshard_layer.py:317-394, :504-721); here the routing is kept
in index form (expert, slot, weight per surviving copy), which is what a gather / grouped-GEMM /
combine pipeline consumes, and the dense tensors are available for checking.

PyTorch implementation (any device); shipped configurations use the dropless router
(``csrc/moe.cu``), this gate serves experiments that need a hard capacity.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class CapacityRouting:
    expert: torch.Tensor     # [S, k] int64, expert of the j-th choice
    slot: torch.Tensor       # [S, k] int64, position in that expert's buffer (valid where keep)
    weight: torch.Tensor     # [S, k] float32, renormalised gate value (0 where dropped)
    keep: torch.Tensor       # [S, k] bool
    capacity: int
    aux_loss: torch.Tensor   # load-balancing loss E^2 * mean(me * ce) of the first choices


def capacity_topk_gating(logits: torch.Tensor, k: int, capacity_factor: float = 1.0, min_capacity: int = 4,
                         valid: int | None = None) -> CapacityRouting:
    S, E = logits.shape
    gates = F.softmax(logits.float(), dim=1)
    cap = max(int(min_capacity), int(math.ceil(capacity_factor * k * S / E)))
    top_v, top_i = torch.topk(gates, k, dim=1)                       # [S, k]
    # admission order: choice-major, then row order (first choices of every token come first)
    flat = top_i.t().reshape(-1)                                      # [k * S]
    onehot = F.one_hot(flat, E)
    loc = (torch.cumsum(onehot, dim=0) - 1).gather(1, flat[:, None]).squeeze(1)
    keep = (loc < cap).view(k, S).t()
    slot = loc.view(k, S).t()
    w = top_v * keep
    w = w / w.sum(dim=1, keepdim=True).clamp_min(torch.finfo(w.dtype).eps)
    n = S if valid is None else valid
    me = gates[:n].mean(dim=0)
    ce = F.one_hot(top_i[:n, 0], E).float().mean(dim=0)
    aux = (me * ce).mean() * E * E
    return CapacityRouting(top_i, slot, w, keep, cap, aux)


def dense_dispatch(r: CapacityRouting, E: int):
    """(combine_weights [S,E,C] float, dispatch_mask [S,E,C] bool): the einsum form."""
    S, k = r.expert.shape
    comb = torch.zeros(S, E, r.capacity, dtype=r.weight.dtype, device=r.weight.device)
    rows = torch.arange(S, device=r.expert.device)[:, None].expand(S, k)
    comb[rows[r.keep], r.expert[r.keep], r.slot[r.keep]] = r.weight[r.keep]
    return comb, comb > 0


def capacity_moe_ffn(x, gate_w, w13, w2, k: int, capacity_factor: float = 1.0, min_capacity: int = 4):
    """Expert FFN with capacity gating: x [S,H], w13 [E,2F,H], w2 [E,H,F]; dropped copies contribute
    nothing (the residual connection around the layer carries the token).  Returns (y, aux_loss)."""
    S, H = x.shape
    E, F2, _ = w13.shape
    Fd = F2 // 2
    r = capacity_topk_gating(F.linear(x.float(), gate_w.float()), k, capacity_factor, min_capacity)
    buf = x.new_zeros(E, r.capacity, H)
    rows = torch.arange(S, device=x.device)[:, None].expand(S, k)
    buf[r.expert[r.keep], r.slot[r.keep]] = x[rows[r.keep]]
    gu = torch.einsum("ech,efh->ecf", buf, w13)
    out = torch.einsum("ecf,ehf->ech", F.silu(gu[..., :Fd]) * gu[..., Fd:], w2)
    y = torch.zeros_like(x, dtype=torch.float32)
    y.index_put_((rows[r.keep],), out[r.expert[r.keep], r.slot[r.keep]].float() * r.weight[r.keep][:, None],
                 accumulate=True)
    return y.to(x.dtype), r.aux_loss
