"""Packed training batch: documents of text / understanding-image / generation-image
segments laid out as one row-major token matrix ``[generation rows | understanding rows]``.

What the reference does in several places is done here once, on the host, while
the batch is collated, so the device step needs no host synchronisation:

* packing order ``[gen | und]`` (pack_two_branch_sequence,
  training/sensenovavl/model/sensenovavl_moe_chat/modeling_sensenovavl_chat_mot.py:324-375),
  here with both partitions padded to 128 rows so that every 128-row tile belongs
  to exactly one branch (``tile_group``);
* (t, h, w) rotary indexes and document ids
  (get_cu_seqlens_and_indexes, training/sensenovavl/data/dataset_interleaved_iterable.py:1626-1728);
* mask inputs doc / pos / image id / flags (create_flex_mask_padding_image_gen, :140-212);
* shifted labels and per-token loss weights (internevo_collate_fn :1735-1947,
  len2weight training/sensenovavl/data/build_dataloader.py:58-67);
* flow-matching timestep per generation image (prepare_image_gen_targets :586-680).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ..config import ModelConfig

KIND_PAD, KIND_TEXT, KIND_UND_IMG, KIND_GEN_IMG = 0, 1, 2, 3
FLAG_GEN, FLAG_BLOCKED = 1, 2
IGNORE = -100
PAD_DOC = 1 << 30


@dataclass
class Segment:
    kind: str                               # "text" | "und_image" | "gen_image"
    ids: Optional[torch.Tensor] = None      # text: int64 [n]
    loss: bool = False                      # text: tokens are prediction targets; image: its <img> token is
    pixels: Optional[torch.Tensor] = None   # image: float [3, H, W] in [-1, 1]
    duplicate_for_und: bool = False         # gen image followed by its clean copy


@dataclass
class Sample:
    segments: List[Segment]
    task: int = 0                           # 3 t2i, 4 editing, 5 interleave (logging only)


def patchify_block_major(pixels: torch.Tensor, patch: int, merge: int):
    """[3,H,W] -> patches [T*merge^2, 3*patch^2] grouped per merged token, plus the
    (column, row) grid position of every patch."""
    C, H, W = pixels.shape
    th, tw = H // (patch * merge), W // (patch * merge)
    x = pixels.reshape(C, th, merge, patch, tw, merge, patch)
    x = x.permute(1, 4, 2, 5, 0, 3, 6).reshape(th * tw * merge * merge, C * patch * patch)
    ty = torch.arange(th).view(th, 1, 1, 1).expand(th, tw, merge, merge)
    tx = torch.arange(tw).view(1, tw, 1, 1).expand(th, tw, merge, merge)
    a = torch.arange(merge).view(1, 1, merge, 1).expand(th, tw, merge, merge)
    b = torch.arange(merge).view(1, 1, 1, merge).expand(th, tw, merge, merge)
    py = (ty * merge + a).reshape(-1).to(torch.int32)
    px = (tx * merge + b).reshape(-1).to(torch.int32)
    return x.contiguous(), px, py, th, tw


def patch_grid_positions(gh: int, gw: int, merge: int):
    """(column, row) of every 16x16 patch of a ``gh x gw`` patch grid in block-major order (the order
    :func:`patchify_block_major` emits: the ``merge x merge`` patches of one token are adjacent)."""
    th, tw = gh // merge, gw // merge
    ty = torch.arange(th).view(th, 1, 1, 1).expand(th, tw, merge, merge)
    tx = torch.arange(tw).view(1, tw, 1, 1).expand(th, tw, merge, merge)
    a = torch.arange(merge).view(1, 1, merge, 1).expand(th, tw, merge, merge)
    b = torch.arange(merge).view(1, 1, 1, merge).expand(th, tw, merge, merge)
    return (tx * merge + b).reshape(-1).to(torch.int32), (ty * merge + a).reshape(-1).to(torch.int32)


def patches_to_tokens(p16: torch.Tensor, patch: int, merge: int) -> torch.Tensor:
    """Block-major patches [T*m*m, 3*p*p] -> token pixels [T, (m p)(m p) 3] in the
    'row, column, channel' order the generation head predicts."""
    T = p16.shape[0] // (merge * merge)
    x = p16.reshape(T, merge, merge, 3, patch, patch)       # T a b c i j
    x = x.permute(0, 1, 4, 2, 5, 3)                          # T a i b j c
    return x.reshape(T, merge * patch * merge * patch * 3)


def tokens_to_patches(tok: torch.Tensor, patch: int, merge: int) -> torch.Tensor:
    T = tok.shape[0]
    x = tok.reshape(T, merge, patch, merge, patch, 3).permute(0, 1, 3, 5, 2, 4)
    return x.reshape(T * merge * merge, 3 * patch * patch)


def apply_time_schedule(t: torch.Tensor, image_seq_len: int, cfg: ModelConfig,
                        timestep_shift: Optional[float] = None) -> torch.Tensor:
    """Shift acts on the noise weight sigma = 1 - t
    (src/sensenova_u1/models/neo_unify/modeling_neo_chat.py:442-462)."""
    sigma = 1 - t
    schedule = cfg.time_schedule if timestep_shift is None else "standard"
    if schedule == "standard":
        s = cfg.timestep_shift if timestep_shift is None else timestep_shift
        sigma = s * sigma / (1 + (s - 1) * sigma)
    elif schedule == "dynamic":
        denom = cfg.max_image_seq_len - cfg.base_image_seq_len
        m = (cfg.max_shift - cfg.base_shift) / denom if denom else 0.0
        mu = image_seq_len * m + (cfg.base_shift - m * cfg.base_image_seq_len) if denom else cfg.base_shift
        if cfg.time_shift_type == "exponential":
            s = math.exp(mu)
            sigma = s * sigma / (1 + (s - 1) * sigma)
        else:
            sigma = mu / (mu + (1 / sigma - 1))
    else:
        raise ValueError(f"unknown time_schedule {schedule}")
    return 1 - sigma


def noise_scale_for(cfg: ModelConfig, image_seq_len: int) -> float:
    ns = cfg.noise_scale
    if cfg.noise_scale_mode in ("resolution", "dynamic"):
        ns = math.sqrt(image_seq_len / float(cfg.noise_scale_base_image_seq_len)) * cfg.noise_scale
    return min(ns, cfg.noise_scale_max_value)


@dataclass
class PackedBatch:
    S: int
    n_gen_pad: int
    ids: torch.Tensor          # [S] int32
    kind: torch.Tensor         # [S] uint8
    meta: torch.Tensor         # [S,4] int32 (doc, pos, img, flags)
    pos3: torch.Tensor         # [3,S] int32 (t, h, w)
    tile_group: torch.Tensor   # [S/128] int32 (0 und, 1 gen, -1 padding-only tile)
    group_range: torch.Tensor  # [2,2] int32: row range [begin,end) of group 0 (und) and 1 (gen)
    labels: torch.Tensor       # [S] int32
    loss_w: torch.Tensor       # [S] float32
    label_rows: torch.Tensor   # [n_label] int64
    text_rows: torch.Tensor    # [n_text] int64
    und_patches: torch.Tensor  # [Pu, patch_dim] bf16/float
    und_px: torch.Tensor
    und_py: torch.Tensor
    und_rows: torch.Tensor     # [Tu] int64
    gen_x16: torch.Tensor      # [Pg, patch_dim] float32 clean pixels, block-major
    gen_px: torch.Tensor
    gen_py: torch.Tensor
    gen_rows: torch.Tensor     # [Tg] int64
    gen_t: torch.Tensor        # [Tg] float32
    gen_ns: torch.Tensor       # [Tg] float32 noise scale
    gen_w: torch.Tensor        # [Tg] float32 loss weight 1/sqrt(len)
    gen_task: torch.Tensor     # [Tg] int32
    n_tokens: int = 0          # real (non padding) tokens
    n_text: int = 0
    n_label: int = 0
    n_samples: int = 0
    ce_weight_sum: float = 0.0
    gen_weight_sum: float = 0.0
    noise_seed: int = 0

    def tensors(self):
        return {k: v for k, v in self.__dict__.items() if isinstance(v, torch.Tensor)}

    def to(self, device, non_blocking=True) -> "PackedBatch":
        kw = dict(self.__dict__)
        for k, v in self.tensors().items():
            kw[k] = v.to(device, non_blocking=non_blocking)
        return PackedBatch(**kw)

    def pin(self) -> "PackedBatch":
        kw = dict(self.__dict__)
        for k, v in self.tensors().items():
            kw[k] = v.pin_memory()
        return PackedBatch(**kw)

    def nbytes(self) -> int:
        return sum(v.numel() * v.element_size() for v in self.tensors().values())


def _round_up(n, a):
    return (n + a - 1) // a * a


def build_packed_batch(samples: Sequence[Sample], cfg: ModelConfig, seq_len: Optional[int] = None,
                       loss_reduction: str = "square", seed: int = 0, img_token_id: int = 1,
                       img_start_id: int = 2, img_end_id: int = 3,
                       patch_dtype=torch.bfloat16) -> PackedBatch:
    """Lays ``samples`` out as one packed sequence.  ``seq_len`` is the padded total
    row count (a multiple of 128; default: the minimum)."""
    gen = torch.Generator().manual_seed(seed)
    patch, merge = cfg.patch_size, cfg.merge_size
    rows = []      # per token: dict-free tuples for speed
    # token fields in original order
    t_ids, t_kind, t_doc, t_pos, t_h, t_w, t_img, t_flags, t_label, t_lw = ([] for _ in range(10))
    und_p, und_px, und_py, gen_p, gen_px, gen_py = [], [], [], [], [], []
    gen_t, gen_ns, gen_w, gen_task = [], [], [], []
    img_counter = 0
    ce_wsum = 0.0
    for d, smp in enumerate(samples):
        start = len(t_ids)
        t = 0
        tok_loss = []   # whether the token itself is a prediction target
        for seg in smp.segments:
            if seg.kind == "text":
                n = int(seg.ids.numel())
                t_ids += seg.ids.tolist()
                t_kind += [KIND_TEXT] * n
                t_pos += list(range(t, t + n))
                t_h += [0] * n
                t_w += [0] * n
                t_img += [0] * n
                t_flags += [0] * n
                tok_loss += [seg.loss] * n
                t += n
            else:
                is_gen = seg.kind == "gen_image"
                copies = [True, False] if (is_gen and seg.duplicate_for_und) else [is_gen]
                p16, px, py, th, tw = patchify_block_major(seg.pixels.float(), patch, merge)
                T = th * tw
                hh = torch.arange(th).view(th, 1).expand(th, tw).reshape(-1).tolist()
                ww = torch.arange(tw).view(1, tw).expand(th, tw).reshape(-1).tolist()
                for ci, as_gen in enumerate(copies):
                    img_counter += 1
                    dup_second = ci == 1
                    # <img>
                    t_ids.append(img_start_id); t_kind.append(KIND_TEXT)
                    t_pos.append(t - 1 if dup_second else t)
                    t_h.append(0); t_w.append(0); t_img.append(0)
                    t_flags.append(FLAG_BLOCKED if dup_second else 0)
                    tok_loss.append(bool(seg.loss) and not dup_second)   # the model learns to open a picture
                    if not dup_second:
                        t += 1
                    t_img_pos = t - 1 if dup_second else t
                    t_ids += [img_token_id] * T
                    t_kind += [KIND_GEN_IMG if as_gen else KIND_UND_IMG] * T
                    t_pos += [t_img_pos] * T
                    t_h += hh; t_w += ww
                    t_img += [img_counter] * T
                    t_flags += [FLAG_GEN if as_gen else 0] * T
                    tok_loss += [False] * T
                    if not dup_second:
                        t += 1
                    # </img>
                    t_ids.append(img_end_id); t_kind.append(KIND_TEXT)
                    t_pos.append(t); t_h.append(0); t_w.append(0); t_img.append(0)
                    blocked = as_gen and len(copies) == 2
                    t_flags.append(FLAG_BLOCKED if blocked else 0)
                    tok_loss.append(False)
                    t += 1
                    if as_gen:
                        gen_p.append(p16); gen_px.append(px); gen_py.append(py)
                        u = torch.randn(1, generator=gen) * cfg.P_std + cfg.P_mean
                        tt = apply_time_schedule(torch.sigmoid(u), T, cfg)
                        gen_t += [float(tt)] * T
                        gen_ns += [noise_scale_for(cfg, T)] * T
                        gen_w += [1.0 / math.sqrt(T)] * T
                        gen_task += [smp.task] * T
                    else:
                        und_p.append(p16); und_px.append(px); und_py.append(py)
        n_doc = len(t_ids) - start
        t_doc += [d] * n_doc
        # shifted labels inside the document
        n_eff = sum(1 for x in tok_loss if x)
        if loss_reduction == "square":
            lw = 1.0 / math.sqrt(max(n_eff, 1))
        elif loss_reduction == "sample":
            lw = 1.0 / max(n_eff, 1)
        else:
            lw = 1.0
        for i in range(n_doc):
            nxt = i + 1
            if nxt < n_doc and tok_loss[nxt]:
                t_label.append(t_ids[start + nxt]); t_lw.append(lw); ce_wsum += lw
            else:
                t_label.append(IGNORE); t_lw.append(0.0)

    n_tok = len(t_ids)
    kind = torch.tensor(t_kind, dtype=torch.uint8)
    is_gen_row = kind == KIND_GEN_IMG
    gen_idx = torch.nonzero(is_gen_row).flatten()
    und_idx = torch.nonzero(~is_gen_row).flatten()
    n_gen, n_und = int(gen_idx.numel()), int(und_idx.numel())
    n_gen_pad = _round_up(n_gen, 128)
    S_min = n_gen_pad + _round_up(n_und, 128)
    S = S_min if seq_len is None else int(seq_len)
    if S % 128 or S < S_min:
        raise ValueError(f"seq_len {S} must be a multiple of 128 and at least {S_min}")
    order = torch.cat([gen_idx, und_idx])                       # original index of each kept row
    dest = torch.cat([torch.arange(n_gen), n_gen_pad + torch.arange(n_und)])

    def scatter(values, fill, dtype):
        out = torch.full((S,), fill, dtype=dtype)
        out[dest] = torch.tensor(values, dtype=dtype)[order]
        return out

    ids = scatter(t_ids, 0, torch.int32)
    kind_s = scatter(t_kind, KIND_PAD, torch.uint8)
    doc = scatter(t_doc, PAD_DOC, torch.int32)
    pos = scatter(t_pos, 0, torch.int32)
    hh = scatter(t_h, 0, torch.int32)
    ww = scatter(t_w, 0, torch.int32)
    img = scatter(t_img, 0, torch.int32)
    flags = scatter(t_flags, FLAG_BLOCKED, torch.int32)
    labels = scatter(t_label, IGNORE, torch.int32)
    loss_w = scatter(t_lw, 0.0, torch.float32)
    meta = torch.stack([doc, pos, img, flags], dim=1).contiguous()
    pos3 = torch.stack([pos, hh, ww], dim=0).contiguous()
    tile_group = torch.full((S // 128,), -1, dtype=torch.int32)
    tile_group[: n_gen_pad // 128] = 1
    tile_group[n_gen_pad // 128: (n_gen_pad + _round_up(n_und, 128)) // 128] = 0
    group_range = torch.tensor([[n_gen_pad, n_gen_pad + _round_up(n_und, 128)], [0, n_gen_pad]],
                               dtype=torch.int32)
    rows_all = torch.arange(S)
    label_rows = rows_all[labels >= 0]
    text_rows = rows_all[kind_s == KIND_TEXT]
    und_rows = rows_all[kind_s == KIND_UND_IMG]
    gen_rows = rows_all[kind_s == KIND_GEN_IMG]
    pd = cfg.patch_dim

    def cat(lst, dtype, width=None):
        if lst:
            return torch.cat(lst).to(dtype)
        return torch.zeros((0, width) if width else (0,), dtype=dtype)

    return PackedBatch(
        S=S, n_gen_pad=n_gen_pad, ids=ids, kind=kind_s, meta=meta, pos3=pos3, tile_group=tile_group,
        group_range=group_range, labels=labels, loss_w=loss_w, label_rows=label_rows,
        text_rows=text_rows,
        und_patches=cat(und_p, patch_dtype, pd), und_px=cat(und_px, torch.int32),
        und_py=cat(und_py, torch.int32), und_rows=und_rows,
        gen_x16=cat(gen_p, torch.float32, pd), gen_px=cat(gen_px, torch.int32),
        gen_py=cat(gen_py, torch.int32), gen_rows=gen_rows,
        gen_t=torch.tensor(gen_t, dtype=torch.float32), gen_ns=torch.tensor(gen_ns, dtype=torch.float32),
        gen_w=torch.tensor(gen_w, dtype=torch.float32), gen_task=torch.tensor(gen_task, dtype=torch.int32),
        n_tokens=n_tok, n_text=int(text_rows.numel()), n_label=int(label_rows.numel()),
        n_samples=len(samples), ce_weight_sum=float(ce_wsum), gen_weight_sum=float(sum(gen_w)),
        noise_seed=seed)


def context_parallel_tiles(n_tiles: int, world: int, rank: int) -> torch.Tensor:
    """128-row tiles of a packed batch dealt zigzag (0,1,..,W-1,W-1,..,1,0,...) to the ranks of a
    context-parallel group: equal tile counts, and equal causal attention work when positions
    grow along the rows."""
    if n_tiles % (2 * world):
        raise ValueError(f"{n_tiles} tiles do not deal evenly to {world} ranks (need a multiple of {2 * world})")
    i = torch.arange(n_tiles)
    m = i % (2 * world)
    owner = torch.where(m < world, m, 2 * world - 1 - m)
    return i[owner == rank]


def split_context_parallel(b: PackedBatch, world: int, rank: int, cfg: ModelConfig) -> PackedBatch:
    """The rows of ``b`` that rank ``rank`` of a context-parallel group holds: whole 128-row tiles,
    dealt zigzag, in ascending order (so the local layout is again [generation | understanding |
    padding]).  Documents span ranks; masks, rotary indexes and shifted labels were computed on the
    whole batch and travel with their rows.  The per-image side arrays are cut to the local tokens."""
    if world == 1:
        return b
    tiles = context_parallel_tiles(b.S // 128, world, rank)
    rows = (tiles[:, None] * 128 + torch.arange(128)[None, :]).reshape(-1).to(b.ids.device)
    S = rows.numel()
    tg = b.tile_group[tiles]
    n_gen_pad = int((tg == 1).sum()) * 128
    n_und_pad = int((tg == 0).sum()) * 128
    kind = b.kind[rows]
    labels = b.labels[rows]
    ar = torch.arange(S, device=rows.device)
    m2 = cfg.merge_size ** 2

    def per_token(global_rows, values, width=1):
        """Selects the entries of a per-image-token array (``width`` consecutive entries per token,
        in the order of ``global_rows``) that belong to local rows, in local row order."""
        if global_rows.numel() == 0:
            return values
        pos = torch.full((b.S,), -1, dtype=torch.long, device=rows.device)
        pos[global_rows] = torch.arange(global_rows.numel(), device=rows.device)
        loc = pos[rows]
        loc = loc[loc >= 0]
        if width == 1:
            return values[loc]
        idx = (loc[:, None] * width + torch.arange(width, device=rows.device)[None, :]).reshape(-1)
        return values[idx]

    gen_w = per_token(b.gen_rows, b.gen_w)
    loss_w = b.loss_w[rows]
    return PackedBatch(
        S=S, n_gen_pad=n_gen_pad, ids=b.ids[rows], kind=kind, meta=b.meta[rows].contiguous(),
        pos3=b.pos3[:, rows].contiguous(), tile_group=tg.contiguous(),
        group_range=torch.tensor([[n_gen_pad, n_gen_pad + n_und_pad], [0, n_gen_pad]], dtype=torch.int32,
                                 device=b.group_range.device),
        labels=labels, loss_w=loss_w, label_rows=ar[labels >= 0], text_rows=ar[kind == KIND_TEXT],
        und_patches=per_token(b.und_rows, b.und_patches, m2), und_px=per_token(b.und_rows, b.und_px, m2),
        und_py=per_token(b.und_rows, b.und_py, m2), und_rows=ar[kind == KIND_UND_IMG],
        gen_x16=per_token(b.gen_rows, b.gen_x16, m2), gen_px=per_token(b.gen_rows, b.gen_px, m2),
        gen_py=per_token(b.gen_rows, b.gen_py, m2), gen_rows=ar[kind == KIND_GEN_IMG],
        gen_t=per_token(b.gen_rows, b.gen_t), gen_ns=per_token(b.gen_rows, b.gen_ns), gen_w=gen_w,
        gen_task=per_token(b.gen_rows, b.gen_task),
        n_tokens=int((kind != KIND_PAD).sum()), n_text=int((kind == KIND_TEXT).sum()),
        n_label=int((labels >= 0).sum()), n_samples=b.n_samples,
        ce_weight_sum=float(loss_w[labels >= 0].sum()), gen_weight_sum=float(gen_w.sum()),
        noise_seed=b.noise_seed * 8191 + rank)
