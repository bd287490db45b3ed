"""Tensor parallelism inside the CUDA training engine (the reference's Megatron "mtp" mode:
column-parallel q/k/v and gate/up projections, row-parallel output and down projections, an all-reduce
after every row-parallel product and after the input gradient of every column-parallel product:
training/sensenovalm/core/parallel/comm/tensor.py:94-146, model/modules/linear.py:665-735).

How it maps onto this engine:

* A tensor-parallel rank runs the ordinary engine on a *local* model configuration with
  ``heads / t`` query heads, ``kv_heads / t`` key/value heads and ``ffn / t`` hidden FFN units
  (:func:`tp_local_config`).  With the fused ``[q | k | v]`` and ``[gate | up]`` weight layouts this is
  exactly the column split of those projections and the row split (of the input dimension) of
  ``wo`` / ``w2``.  Everything else (embeddings, norms, pixel front-ends, heads) is replicated and
  sees replicated activations, so its gradients are identical on every rank of the group.
* The four partial sums per layer and pass are completed by :class:`PeerAllReduce`: a two-shot
  all-reduce over NVLink peer memory made of this package's kernels (``rs_pull``: each rank sums its
  piece from every peer's staging buffer; ``wp_gather``: every rank collects all reduced pieces),
  ordered by flag barriers in symmetric memory with bounded waits.  The residual is added by rank 0's
  GEMM epilogue only, so the all-reduce also completes ``x + attention`` / ``x + ffn`` without a
  further pass.
* :func:`shard_store_tp` cuts a full :class:`ParamStore` into the local one (and
  :func:`merge_tp_stores` reassembles it for checkpoints / exports).
"""
from __future__ import annotations

from typing import List, Sequence

import torch
import torch.distributed as dist

from ..config import ModelConfig
from ..models.params import ParamStore


def tp_local_config(cfg: ModelConfig, t: int) -> ModelConfig:
    if t == 1:
        return cfg
    if cfg.is_moe:
        raise NotImplementedError("tensor parallel covers the dense model")
    if cfg.num_heads % t or cfg.num_kv_heads % t or cfg.ffn_size % (t * 128):
        raise ValueError(f"heads {cfg.num_heads}, kv heads {cfg.num_kv_heads} and FFN {cfg.ffn_size} must split over "
                         f"{t} tensor-parallel ranks (FFN in multiples of 128)")
    return cfg.replace(num_heads=cfg.num_heads // t, num_kv_heads=cfg.num_kv_heads // t, ffn_size=cfg.ffn_size // t)


def _slices(cfg: ModelConfig, t: int, r: int):
    """Row / column index ranges of rank ``r`` inside the full fused tensors."""
    qd, kd, F = cfg.q_dim, cfg.kv_dim, cfg.ffn_size
    ql, kl, fl = qd // t, kd // t, F // t
    qkv_rows = torch.cat([torch.arange(r * ql, (r + 1) * ql), qd + torch.arange(r * kl, (r + 1) * kl),
                          qd + kd + torch.arange(r * kl, (r + 1) * kl)])
    w13_rows = torch.cat([torch.arange(r * fl, (r + 1) * fl), F + torch.arange(r * fl, (r + 1) * fl)])
    return qkv_rows, w13_rows, slice(r * ql, (r + 1) * ql), slice(r * fl, (r + 1) * fl)


def _layer_prefixes(cfg: ModelConfig) -> List[str]:
    return [f"layers.{l}." for l in range(cfg.num_layers)] + [f"mtp.{k}.layer." for k in range(cfg.num_mtp_layers)]


def shard_store_tp(full: ParamStore, t: int, r: int, device=None, with_grads: bool = True, **kw) -> ParamStore:
    """The tensor-parallel rank ``r`` of ``t``'s share of ``full`` as a store of the local configuration."""
    cfg = full.cfg
    loc = ParamStore(tp_local_config(cfg, t), device=device or full.device, dtype=full.dtype, with_grads=with_grads, **kw)
    qkv_rows, w13_rows, o_cols, f_cols = _slices(cfg, t, r)
    sharded = set()
    for s in _layer_prefixes(cfg):
        dev = full.device
        loc.p[s + "wqkv"].copy_(full.p[s + "wqkv"].index_select(1, qkv_rows.to(dev)))
        loc.p[s + "w13"].copy_(full.p[s + "w13"].index_select(1, w13_rows.to(dev)))
        loc.p[s + "wo"].copy_(full.p[s + "wo"][:, :, o_cols])
        loc.p[s + "w2"].copy_(full.p[s + "w2"][:, :, f_cols])
        sharded.update(s + n for n in ("wqkv", "w13", "wo", "w2"))
    for name, v in full.p.items():
        if name not in sharded:
            loc.p[name].copy_(v)
    return loc


def merge_tp_stores(parts: Sequence[ParamStore], cfg: ModelConfig, device="cpu") -> ParamStore:
    """Inverse of :func:`shard_store_tp` (weights only)."""
    t = len(parts)
    full = ParamStore(cfg, device=device, dtype=parts[0].dtype, with_grads=False)
    sharded = set()
    for s in _layer_prefixes(cfg):
        for r, part in enumerate(parts):
            qkv_rows, w13_rows, o_cols, f_cols = _slices(cfg, t, r)
            full.p[s + "wqkv"].index_copy_(1, qkv_rows.to(device), part.p[s + "wqkv"].to(device))
            full.p[s + "w13"].index_copy_(1, w13_rows.to(device), part.p[s + "w13"].to(device))
            full.p[s + "wo"][:, :, o_cols] = part.p[s + "wo"].to(device)
            full.p[s + "w2"][:, :, f_cols] = part.p[s + "w2"].to(device)
        sharded.update(s + n for n in ("wqkv", "w13", "wo", "w2"))
    for name, v in parts[0].p.items():
        if name not in sharded:
            full.p[name].copy_(v.to(device))
    return full


class PeerAllReduce:
    """In-place sum of a bf16 tensor over the ranks of ``group`` by peer loads (two-shot: reduce-scatter pull +
    all-gather pull).  Two flag barriers per call: "every rank's addend is staged" and "every piece is reduced";
    stream order on each rank makes buffer reuse by the next call safe (a rank reaches the next call's first barrier
    only after its gather of this call, and passes this call's second barrier only after its pull)."""

    def __init__(self, group, device, max_numel: int):
        from .symm import FlagBarrier, SymmetricBuffer
        self.group, self.dev = group, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if max_numel % (8 * self.world):
            max_numel += 8 * self.world - max_numel % (8 * self.world)
        self.max_numel = max_numel
        self.stage = SymmetricBuffer(max_numel, torch.bfloat16, self.dev, group)
        self.red = SymmetricBuffer(max_numel // self.world, torch.bfloat16, self.dev, group)
        self.bar = FlagBarrier(group, self.dev)
        self.calls = 0

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        from ..ops import _lib
        from ..ops._lib import c_int, c_ll, c_void_p
        n = t.numel()
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or n % (8 * self.world) or n > self.max_numel:
            raise ValueError(f"all_reduce_: contiguous bf16 tensor of a multiple of {8 * self.world} elements, at most "
                             f"{self.max_numel} (got {t.dtype}, {n})")
        per = n // self.world
        st = c_void_p(torch.cuda.current_stream().cuda_stream)
        self.stage.tensor[:n].copy_(t.view(-1))
        self.bar.barrier()
        _lib.call("rs_pull", self.stage.c_ptrs, c_int(self.world), c_ll(self.rank * per), c_ll(per),
                  c_void_p(self.red.tensor.data_ptr()), c_int(0), c_void_p(None), c_int(0), st)
        self.bar.barrier()
        _lib.call("wp_gather", self.red.c_ptrs, c_int(self.world), c_ll(0), c_ll(per), c_void_p(t.data_ptr()),
                  c_int(296), st)
        self.calls += 1
        return t
