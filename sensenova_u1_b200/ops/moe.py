"""Python faces of the MoE routing kernels (csrc/moe.cu)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from ._lib import c_float, c_int, c_void_p

P = lambda t: c_void_p(_lib.ptr(t))
ST = lambda: c_void_p(_lib.stream())


@dataclass
class Routing:
    R: int
    E: int
    K: int
    probs: torch.Tensor       # [R,E] fp32
    top_idx: torch.Tensor     # [R,K] int32 (-1: row not routed)
    top_w: torch.Tensor       # [R,K] fp32
    counts: torch.Tensor      # [E] int32
    seg_start: torch.Tensor   # [E] int32, 128-aligned
    seg_end: torch.Tensor     # [E] int32 (padded end)
    tile_group: torch.Tensor  # [max_tiles] int32
    total_rows: torch.Tensor  # [1] int32
    dest: torch.Tensor        # [R,K] int32 row in the permuted buffer
    max_rows: int
    lse: torch.Tensor = None          # [R] fp32 row log-sum-exp (z-loss), when asked for
    row_class: torch.Tensor = None    # [R] int32 token class (0 text, 1 image), when given
    class_counts: torch.Tensor = None  # [2,E] int32 routed slots per class


def max_permuted_rows(R: int, K: int, E: int) -> int:
    return (R * K + E * 127 + 127) // 128 * 128


def route(logits: torch.Tensor, K: int, norm_topk: bool = True, row_valid=None, bufs=None,
          layout: bool = True, sel_bias=None, want_lse: bool = False, row_class=None) -> Routing:
    """Softmax gate, top-k, renormalise, count, and (``layout``) lay tokens out in expert segments
    padded to 128 rows; all on the device, nothing is read back.  ``layout=False`` stops after the
    counts (expert parallelism derives the layout from every rank's counts instead)."""
    R, E = logits.shape
    dev = logits.device
    max_rows = max_permuted_rows(R, K, E)
    mt = max_rows // 128
    mk = (lambda name, shape, dt: bufs.get(name, shape, dt)) if bufs is not None else \
        (lambda name, shape, dt: torch.empty(shape, dtype=dt, device=dev))
    probs = mk("moe.probs", (R, E), torch.float32)
    top_idx = mk("moe.idx", (R, K), torch.int32)
    top_w = mk("moe.w", (R, K), torch.float32)
    counts = mk("moe.counts", (E,), torch.int32)
    counts.zero_()
    seg_start = mk("moe.ss", (E,), torch.int32)
    seg_end = mk("moe.se", (E,), torch.int32)
    tile_group = mk("moe.tg", (mt,), torch.int32)
    total = mk("moe.tot", (1,), torch.int32)
    dest = mk("moe.dest", (R, K), torch.int32)
    if sel_bias is None and not want_lse and row_class is None:
        _lib.call("moe_route", P(logits), c_int(R), c_int(E), c_int(K), c_int(1 if norm_topk else 0), P(probs),
                  P(top_idx), P(top_w), P(counts), P(row_valid), c_int(mt if layout else 0), P(seg_start), P(seg_end),
                  P(tile_group), P(total), P(dest), ST())
        return Routing(R, E, K, probs, top_idx, top_w, counts, seg_start, seg_end, tile_group, total, dest, max_rows)
    # training extras (csrc/moe.cu::snu1_moe_route_ex): selection bias of bias-based balancing, row log-sum-exp for
    # the z-loss, routed slots per token class for the class-weighted balance loss
    lse = mk("moe.lse", (R,), torch.float32) if want_lse else None
    cc = None
    if row_class is not None:
        cc = mk("moe.ccounts", (2, E), torch.int32)
        cc.zero_()
    _lib.call("moe_route_ex", P(logits), c_int(R), c_int(E), c_int(K), c_int(1 if norm_topk else 0), P(probs),
              P(top_idx), P(top_w), P(counts), P(row_valid), c_int(mt if layout else 0), P(seg_start), P(seg_end),
              P(tile_group), P(total), P(dest), P(sel_bias), P(lse), P(row_class), P(cc), ST())
    return Routing(R, E, K, probs, top_idx, top_w, counts, seg_start, seg_end, tile_group, total, dest, max_rows,
                   lse, row_class, cc)


def gather(x, r: Routing, xp):
    _lib.call("moe_gather", P(x), P(r.dest), P(r.top_idx), P(xp), c_int(r.R), c_int(r.K), c_int(x.shape[1]), ST())
    return xp


def combine(yp, r: Routing, residual, y):
    _lib.call("moe_combine", P(yp), P(r.dest), P(r.top_idx), P(r.top_w), P(residual), P(y), c_int(r.R),
              c_int(r.K), c_int(y.shape[1]), ST())
    return y


def combine_bwd(dy, yp, r: Routing, dyp, dw):
    _lib.call("moe_combine_bwd", P(dy), P(yp), P(r.dest), P(r.top_idx), P(r.top_w), P(dyp), P(dw), c_int(r.R),
              c_int(r.K), c_int(dy.shape[1]), ST())


def gather_bwd(dxp, r: Routing, dx, accumulate=False):
    _lib.call("moe_gather_bwd", P(dxp), P(r.dest), P(r.top_idx), P(dx), c_int(1 if accumulate else 0), c_int(r.R),
              c_int(r.K), c_int(dx.shape[1]), ST())


def router_bwd(r: Routing, dw, aux_scale: float, norm_topk: bool, dlogits, class_scales=None, z_scale: float = 0.0):
    """``class_scales = (text, image)``: per-class balance-loss gradient scales (needs ``r.class_counts``);
    ``z_scale``: z-loss coefficient / valid rows (needs ``r.lse``)."""
    if class_scales is None and z_scale == 0.0:
        _lib.call("moe_router_bwd", P(r.probs), P(r.top_idx), P(r.top_w), P(dw), P(r.counts), c_float(aux_scale),
                  c_int(1 if norm_topk else 0), P(dlogits), c_int(r.R), c_int(r.E), c_int(r.K), ST())
        return dlogits
    use_c = class_scales is not None and r.class_counts is not None
    c0, c1 = class_scales if use_c else (0.0, 0.0)
    _lib.call("moe_router_bwd_ex", P(r.probs), P(r.top_idx), P(r.top_w), P(dw), P(r.counts), c_float(aux_scale),
              c_int(1 if norm_topk else 0), P(dlogits), c_int(r.R), c_int(r.E), c_int(r.K),
              P(r.row_class if use_c else None), P(r.class_counts if use_c else None), c_float(c0), c_float(c1),
              P(r.lse if z_scale != 0.0 else None), c_float(z_scale), ST())
    return dlogits


# ---------------------------------------------------------------------------------------------
# Expert parallelism over NVLink peer memory (csrc/moe.cu, second half)
# ---------------------------------------------------------------------------------------------
@dataclass
class EpRouting:
    """Layout of one mixture under expert parallelism.  ``dest`` indexes rows of the OWNER's receive
    buffer (owner of global expert e = e // E_loc); the segment tables describe this rank's own
    receive buffer (its E_loc experts, rows of all source ranks)."""
    R: int
    E: int
    K: int
    E_loc: int
    world: int
    top_idx: torch.Tensor
    top_w: torch.Tensor
    dest: torch.Tensor
    base: torch.Tensor
    seg_start: torch.Tensor
    seg_end: torch.Tensor
    seg_fill: torch.Tensor     # [E_loc] first padding row of every local segment
    tile_group: torch.Tensor
    total_rows: torch.Tensor
    max_rows: int


def ep_put_counts(counts, counts_all_ptrs, world: int, rank: int, E: int):
    _lib.call("moe_ep_put_counts", P(counts), counts_all_ptrs, c_int(world), c_int(rank), c_int(E), ST())


def ep_plan(counts_all, world: int, rank: int, E: int, max_rows: int, top_idx, top_w, R: int, K: int, bufs) -> EpRouting:
    dev = counts_all.device
    mt = max_rows // 128
    E_loc = E // world
    base = bufs.get("ep.base", (E,), torch.int32)
    ss = bufs.get("ep.ss", (E_loc,), torch.int32)
    se = bufs.get("ep.se", (E_loc,), torch.int32)
    sf = bufs.get("ep.sf", (E_loc,), torch.int32)
    tg = bufs.get("ep.tg", (mt,), torch.int32)
    tot = bufs.get("ep.tot", (1,), torch.int32)
    dest = bufs.get("ep.dest", (max(R, 1), K), torch.int32)
    _lib.call("moe_ep_plan", P(counts_all), c_int(world), c_int(rank), c_int(E), c_int(mt), P(base), P(ss), P(se), P(sf),
              P(tg), P(tot), P(top_idx) if R > 0 else c_void_p(None), c_int(R * K), P(dest), ST())
    return EpRouting(R, E, K, E_loc, world, top_idx, top_w, dest, base, ss, se, sf, tg, tot, max_rows)


def ep_zero_pads(r: EpRouting, a, b=None):
    """Clears the padding rows of the receive buffers ``a`` / ``b`` ([max_rows, H]) of this rank."""
    _lib.call("moe_ep_zero_pads", P(a), P(b), P(r.seg_fill), P(r.seg_end), c_int(r.E_loc), c_int(a.shape[1]),
              c_int(r.max_rows), ST())


def ep_dispatch(x, r: EpRouting, xp_ptrs):
    if r.R > 0:
        _lib.call("moe_ep_dispatch", P(x), P(r.dest), P(r.top_idx), xp_ptrs, c_int(r.world), c_int(r.E_loc),
                  c_int(r.R), c_int(r.K), c_int(x.shape[1]), c_int(r.max_rows), ST())


def ep_combine(yp_ptrs, r: EpRouting, weights, residual, y):
    """y = residual + sum_k w_k * yp_owner[dest_k]; ``weights=None`` sums with weight 1 (the backward of
    dispatch), ``residual=None`` starts from zero."""
    if r.R > 0:
        _lib.call("moe_ep_combine", yp_ptrs, c_int(r.world), P(r.dest), P(r.top_idx), P(weights), P(residual), P(y),
                  c_int(r.E_loc), c_int(r.R), c_int(r.K), c_int(y.shape[1]), c_int(r.max_rows), ST())
    return y


def ep_combine_bwd(dy, yp_ptrs, dyp_ptrs, r: EpRouting, dw):
    if r.R > 0:
        _lib.call("moe_ep_combine_bwd", P(dy), yp_ptrs, dyp_ptrs, c_int(r.world), P(r.dest), P(r.top_idx),
                  P(r.top_w), P(dw), c_int(r.E_loc), c_int(r.R), c_int(r.K), c_int(dy.shape[1]), c_int(r.max_rows), ST())
