"""Packed mixed-mask attention (csrc/attn_fwd_sm100.cu, csrc/attn_bwd_sm100.cu).

Token metadata is an int32 tensor ``[S, 4]`` = (doc, pos, img, flags) with
``flags`` bit0 = generation-branch token, bit1 = key that nobody may attend to.
The mask rule is documented in ``csrc/attn_common.cuh`` and restated by
:func:`dense_mask` (the PyTorch oracle used by the tests; it follows
training/sensenovavl/model/sensenovavl_moe_chat/modeling_sensenovavl_chat_mot.py:140-212).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from ._lib import c_float, c_int, c_ll, c_void_p

FLAG_GEN = 1
FLAG_BLOCKED = 2


def make_meta(doc, pos, img=None, gen=None, blocked=None) -> torch.Tensor:
    """Packs per-token mask inputs into the ``[S,4]`` int32 record the kernels read."""
    doc = doc.to(torch.int32)
    z = torch.zeros_like(doc)
    img = z if img is None else img.to(torch.int32)
    flags = z.clone()
    if gen is not None:
        flags = flags | (gen.to(torch.int32) * FLAG_GEN)
    if blocked is not None:
        flags = flags | (blocked.to(torch.int32) * FLAG_BLOCKED)
    return torch.stack([doc, pos.to(torch.int32), img, flags], dim=1).contiguous()


def dense_mask(meta_q: torch.Tensor, meta_k: torch.Tensor) -> torch.Tensor:
    """Boolean ``[Sq,Sk]`` mask, True = may attend (oracle; any device)."""
    dq, pq, iq, fq = [meta_q[:, i, None] for i in range(4)]
    dk, pk, ik, fk = [meta_k[None, :, i] for i in range(4)]
    gen_q, gen_k = (fq & FLAG_GEN) != 0, (fk & FLAG_GEN) != 0
    same_img = (iq > 0) & (iq == ik)
    base = (dq == dk) & ((pq >= pk) | same_img)
    gate1 = (~gen_k) | (gen_q & (iq == ik))
    gate2 = (~gen_q) | gen_k | (pk != pq)
    return base & gate1 & gate2 & ((fk & FLAG_BLOCKED) == 0)


def reference_attention(q, k, v, meta_q, meta_k, scale):
    """fp32 dense masked softmax attention.  q ``[Sq,Hq,D]``, k/v ``[Sk,Hkv,D]``."""
    Sq, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    qf = q.float().transpose(0, 1)
    kf = k.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    vf = v.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    s = torch.einsum("hqd,hkd->hqk", qf, kf) * scale
    mask = dense_mask(meta_q, meta_k)
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)  # rows without any key give zeros
    return torch.einsum("hqk,hkd->hqd", p, vf).transpose(0, 1)


@dataclass
class TilePlan:
    """Device-side classification of (query tile, key tile) pairs, built once per
    packed batch and shared by every layer and by forward and backward."""
    meta_q: torch.Tensor
    meta_k: torch.Tensor
    Sq: int
    Sk: int
    cls: torch.Tensor
    kv_list: torch.Tensor
    kv_count: torch.Tensor
    q_list: torch.Tensor
    q_count: torch.Tensor
    pair_list: torch.Tensor
    pair_count: torch.Tensor
    # mask bits of the partial (query tile, key tile) pairs, in both orientations (None: the kernels evaluate
    # the mask rule per element on partial tiles)
    tile_slot: torch.Tensor | None = None
    bits_q: torch.Tensor | None = None
    bits_k: torch.Tensor | None = None
    slot_counter: torch.Tensor | None = None
    # launch orders, longest tile list first (None: natural order)
    pair_order: torch.Tensor | None = None
    q_order: torch.Tensor | None = None
    kv_order: torch.Tensor | None = None

    def _mask_ptrs(self):
        if self.tile_slot is None:
            return c_void_p(None), c_void_p(None), c_void_p(None)
        return c_void_p(self.tile_slot.data_ptr()), c_void_p(self.bits_q.data_ptr()), c_void_p(self.bits_k.data_ptr())


def _optr(t):
    return c_void_p(None if t is None else t.data_ptr())


def mask_slot_capacity(nq: int, nk: int) -> int:
    """Slots for partial pairs: packed batches have a few per tile row (diagonals, document and image borders),
    never more than there are pairs.  A pair beyond the capacity falls back to the per-element rule."""
    return min(nq * nk, 16 * (nq + nk) + 64)


def build_plan(meta_q: torch.Tensor, meta_k: torch.Tensor | None = None, mask_slots: int | None = None) -> TilePlan:
    """``mask_slots``: capacity of the mask-bit table (default :func:`mask_slot_capacity`; 0 = no table)."""
    if meta_k is None:
        meta_k = meta_q
    for m in (meta_q, meta_k):
        if not (m.is_cuda and m.dtype == torch.int32 and m.dim() == 2 and m.shape[1] == 4
                and m.is_contiguous()):
            raise ValueError("token metadata must be a contiguous CUDA int32 [S,4] tensor")
    Sq, Sk = meta_q.shape[0], meta_k.shape[0]
    nq, nk = (Sq + 127) // 128, (Sk + 127) // 128
    dev = meta_q.device
    cls = torch.empty(nq, nk, dtype=torch.uint8, device=dev)
    kv_list = torch.empty(nq, nk, dtype=torch.int32, device=dev)
    kv_count = torch.empty(nq, dtype=torch.int32, device=dev)
    q_list = torch.empty(nk, nq, dtype=torch.int32, device=dev)
    q_count = torch.empty(nk, dtype=torch.int32, device=dev)
    npair = (nq + 1) // 2
    pair_list = torch.empty(npair, nk, dtype=torch.int32, device=dev)
    pair_count = torch.empty(npair, dtype=torch.int32, device=dev)
    cap = mask_slot_capacity(nq, nk) if mask_slots is None else int(mask_slots)
    tile_slot = bits_q = bits_k = counter = None
    if cap > 0:
        tile_slot = torch.empty(nq, nk, dtype=torch.int32, device=dev)
        bits_q = torch.empty(cap, 128, 4, dtype=torch.int32, device=dev)
        bits_k = torch.empty(cap, 128, 4, dtype=torch.int32, device=dev)
        counter = torch.empty(1, dtype=torch.int32, device=dev)
    P = lambda t: c_void_p(None if t is None else t.data_ptr())
    _lib.call("attn_build_tiles", c_void_p(meta_q.data_ptr()), c_void_p(meta_k.data_ptr()),
              c_int(Sq), c_int(Sk), c_void_p(cls.data_ptr()), c_void_p(kv_list.data_ptr()),
              c_void_p(kv_count.data_ptr()), c_void_p(q_list.data_ptr()),
              c_void_p(q_count.data_ptr()), c_void_p(pair_list.data_ptr()),
              c_void_p(pair_count.data_ptr()), P(tile_slot), P(bits_q), P(bits_k), c_int(cap), P(counter),
              c_void_p(_lib.stream()))
    plan = TilePlan(meta_q, meta_k, Sq, Sk, cls, kv_list, kv_count, q_list, q_count, pair_list, pair_count,
                    tile_slot, bits_q, bits_k, counter)
    if max(nq, nk) > 1 and not torch.cuda.is_current_stream_capturing():
        # CTAs are dispatched in grid order: the tiles with the longest lists go first, so that the last wave of a
        # packed batch (lists of 3 to 40 tiles) is made of short ones
        order = lambda c: torch.argsort(c, descending=True, stable=True).to(torch.int32)
        plan.pair_order, plan.q_order, plan.kv_order = order(pair_count), order(kv_count), order(q_count)
    return plan


def _check_heads(t, name):
    if not (t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 3 and t.shape[2] == 128
            and t.stride(2) == 1 and t.stride(1) == 128):
        raise ValueError(f"{name} must be CUDA bf16 [S, H, 128] with contiguous heads")


def attention_fwd(q, k, v, plan: TilePlan, scale: float, out=None, lse=None):
    """Returns ``(out [Sq,Hq,128] bf16, lse [Hq,Sq] fp32 in log2 units)``.
    ``q``/``k``/``v`` may be column slices of wider row-major buffers."""
    for t, nme in ((q, "q"), (k, "k"), (v, "v")):
        _check_heads(t, nme)
    Sq, Hq, _ = q.shape
    Sk, Hkv, _ = k.shape
    assert Sq == plan.Sq and Sk == plan.Sk and v.shape[0] == Sk
    if out is None:
        out = torch.empty(Sq, Hq, 128, dtype=torch.bfloat16, device=q.device)
    if lse is None:
        lse = torch.empty(Hq, Sq, dtype=torch.float32, device=q.device)
    _lib.call("attn_fwd", c_void_p(q.data_ptr()), c_ll(q.stride(0)), c_void_p(k.data_ptr()),
              c_ll(k.stride(0)), c_void_p(v.data_ptr()), c_ll(v.stride(0)),
              c_void_p(out.data_ptr()), c_ll(out.stride(0)), c_void_p(lse.data_ptr()),
              c_void_p(plan.meta_q.data_ptr()), c_void_p(plan.meta_k.data_ptr()),
              c_void_p(plan.pair_list.data_ptr()), c_void_p(plan.pair_count.data_ptr()),
              c_int(Sq), c_int(Sk), c_int(Hq), c_int(Hkv), c_float(scale), *plan._mask_ptrs()[:2],
              _optr(plan.pair_order), c_void_p(_lib.stream()))
    return out, lse


def attention_bwd(q, k, v, o, dout, lse, plan: TilePlan, scale: float, dq=None, dk=None, dv=None,
                  delta=None):
    """Gradients of :func:`attention_fwd`.  ``dq``/``dk``/``dv`` may be column
    slices of one wider buffer (for instance the gradient of a fused QKV projection)."""
    for t, nme in ((q, "q"), (k, "k"), (v, "v"), (o, "o"), (dout, "dout")):
        _check_heads(t, nme)
    Sq, Hq, _ = q.shape
    Sk, Hkv, _ = k.shape
    dev = q.device
    if dq is None:
        dq = torch.empty(Sq, Hq, 128, dtype=torch.bfloat16, device=dev)
    if dk is None:
        dk = torch.empty(Sk, Hkv, 128, dtype=torch.bfloat16, device=dev)
    if dv is None:
        dv = torch.empty(Sk, Hkv, 128, dtype=torch.bfloat16, device=dev)
    for t, nme in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        _check_heads(t, nme)
    if delta is None:
        delta = torch.empty(Hq, Sq, dtype=torch.float32, device=dev)
    _lib.call("attn_bwd", c_void_p(q.data_ptr()), c_ll(q.stride(0)), c_void_p(k.data_ptr()),
              c_ll(k.stride(0)), c_void_p(v.data_ptr()), c_ll(v.stride(0)),
              c_void_p(o.data_ptr()), c_ll(o.stride(0)), c_void_p(dout.data_ptr()),
              c_ll(dout.stride(0)), c_void_p(lse.data_ptr()), c_void_p(delta.data_ptr()),
              c_void_p(dq.data_ptr()), c_ll(dq.stride(0)), c_void_p(dk.data_ptr()),
              c_ll(dk.stride(0)), c_void_p(dv.data_ptr()), c_ll(dv.stride(0)),
              c_void_p(plan.meta_q.data_ptr()), c_void_p(plan.meta_k.data_ptr()),
              c_void_p(plan.kv_list.data_ptr()), c_void_p(plan.kv_count.data_ptr()),
              c_void_p(plan.q_list.data_ptr()), c_void_p(plan.q_count.data_ptr()),
              c_int(Sq), c_int(Sk), c_int(Hq), c_int(Hkv), c_float(scale), *plan._mask_ptrs(),
              _optr(plan.q_order), _optr(plan.kv_order), c_void_p(_lib.stream()))
    return dq, dk, dv
