"""Plain PyTorch statement of the NEO-unify MoT training math.

This is the numerical oracle of the framework: it runs on any device and dtype
under torch autograd, consumes the same :class:`ParamStore` and
:class:`PackedBatch` as the CUDA engine, and is what the CPU / gloo tests train
with.  It follows the reference modelling code:

* decoder layer with per-branch weights: training/sensenovalm/model/modeling_qwen3_moe_mot.py:306-396
* q/k half-head RMSNorm + t/h/w RoPE: src/sensenova_u1/models/neo_unify/modeling_qwen3.py:444-468
* patch front-end: src/sensenova_u1/models/neo_unify/modeling_neo_vit.py:112-204
* timestep embedder / fm head: src/sensenova_u1/models/neo_unify/modeling_fm_modules.py:23-60,
  modeling_neo_chat.py:170-270
* losses: training/sensenovavl/model/sensenovavl_moe_chat/modeling_sensenovavl_chat_mot.py:1403-1480,
  training/sensenovalm/model/losses/ce_loss.py:19-84
* MoE block: src/sensenova_u1/models/neo_unify/modeling_qwen3_moe.py:51-119
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from ..data.batch import KIND_GEN_IMG, PackedBatch, patches_to_tokens
from .params import GEN, UND


def rmsnorm(x, g, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * g


def rope_inv_freq(cfg: ModelConfig, device):
    """t axis: base^(-2j/(D/2)) for j < D/4; h, w axes: base_hw^(-2j/(D/4)) for j < D/8
    (the "keep frequency range" rule: computed for twice the width, every other entry)."""
    D = cfg.head_dim
    nt, nhw = D // 4, D // 8
    inv_t = 1.0 / (cfg.rope_base ** (torch.arange(0, 2 * nt, 2, dtype=torch.float32, device=device) / (D / 2)))
    inv_hw = 1.0 / (cfg.rope_base_hw ** (torch.arange(0, 2 * nhw, 2, dtype=torch.float32, device=device) / (D / 4)))
    return inv_t, inv_hw


def _rot_half(x):
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def rope3d(x, pos3, cfg: ModelConfig):
    """x [S, heads, D]; pos3 [3, S]."""
    D = cfg.head_dim
    inv_t, inv_hw = rope_inv_freq(cfg, x.device)
    parts, widths = [], [D // 2, D // 4, D // 4]
    off = 0
    for axis, (wd, inv) in enumerate(zip(widths, [inv_t, inv_hw, inv_hw])):
        fr = pos3[axis].float()[:, None] * inv[None, :]
        emb = torch.cat([fr, fr], dim=-1)[:, None, :]
        xs = x[..., off:off + wd].float()
        parts.append(xs * emb.cos() + _rot_half(xs) * emb.sin())
        off += wd
    return torch.cat(parts, dim=-1).to(x.dtype)


def qk_norm_rope(qkv, gains, pos3, cfg: ModelConfig):
    """qkv [S, q_dim + 2 kv_dim] -> q [S,Hq,D], k [S,Hkv,D], v [S,Hkv,D]; gains [4, D/2]."""
    S = qkv.shape[0]
    D, Hq, Hk = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    q = qkv[:, :cfg.q_dim].view(S, Hq, D)
    k = qkv[:, cfg.q_dim:cfg.q_dim + cfg.kv_dim].view(S, Hk, D)
    v = qkv[:, cfg.q_dim + cfg.kv_dim:].view(S, Hk, D)
    h = D // 2
    q = torch.cat([rmsnorm(q[..., :h], gains[0], cfg.rms_eps), rmsnorm(q[..., h:], gains[1], cfg.rms_eps)], -1)
    k = torch.cat([rmsnorm(k[..., :h], gains[2], cfg.rms_eps), rmsnorm(k[..., h:], gains[3], cfg.rms_eps)], -1)
    return rope3d(q, pos3, cfg), rope3d(k, pos3, cfg), v


def dense_mask(meta_q, meta_k):
    from ..ops.attention import dense_mask as dm
    return dm(meta_q, meta_k)


def attention(q, k, v, mask, scale):
    Hq, Hk = q.shape[1], k.shape[1]
    rep = Hq // Hk
    qf = q.float().transpose(0, 1)
    kf = k.float().transpose(0, 1).repeat_interleave(rep, 0)
    vf = v.float().transpose(0, 1).repeat_interleave(rep, 0)
    s = torch.einsum("hqd,hkd->hqk", qf, kf) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
    return torch.einsum("hqk,hkd->hqd", p, vf).transpose(0, 1).to(q.dtype)


def _branch(x, w_pair, is_gen_row, fn):
    """Applies fn(x, w[branch]) per row by branch (both evaluated, then selected)."""
    yu, yg = fn(x, w_pair[UND]), fn(x, w_pair[GEN])
    return torch.where(is_gen_row[:, None], yg, yu)


def moe_ffn(x, gate_w, w13, w2, top_k, norm_topk):
    """Dropless top-k mixture: fp32 softmax gate, renormalised top-k weights."""
    logits = F.linear(x.float(), gate_w.float())
    probs = torch.softmax(logits, dim=-1)
    tw, ti = torch.topk(probs, top_k, dim=-1)
    if norm_topk:
        tw = tw / tw.sum(-1, keepdim=True)
    out = torch.zeros_like(x, dtype=torch.float32)
    Fe = w2.shape[-1]
    for e in range(gate_w.shape[0]):
        sel = (ti == e)
        rows = sel.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        xe = x[rows]
        gu = F.linear(xe, w13[e])
        act = F.silu(gu[:, :Fe]) * gu[:, Fe:]
        ye = F.linear(act, w2[e]).float()
        we = (tw[rows] * sel[rows]).sum(-1, keepdim=True)
        out.index_add_(0, rows, ye * we)
    return out.to(x.dtype), logits


def decoder_layer(p: Dict[str, torch.Tensor], l, x, is_gen_row, pos3, mask, cfg: ModelConfig,
                  aux: Optional[list] = None):
    """``l``: layer index, or a full name prefix (e.g. ``"mtp.0.layer."``)."""
    s = l if isinstance(l, str) else f"layers.{l}."
    eps = cfg.rms_eps
    h = torch.where(is_gen_row[:, None], rmsnorm(x, p[s + "attn_norm"][GEN], eps),
                    rmsnorm(x, p[s + "attn_norm"][UND], eps))
    qkv = _branch(h, p[s + "wqkv"], is_gen_row, F.linear)
    qu, ku, vu = qk_norm_rope(qkv, p[s + "qk_norm"][UND], pos3, cfg)
    qg, kg, _ = qk_norm_rope(qkv, p[s + "qk_norm"][GEN], pos3, cfg)
    sel = is_gen_row[:, None, None]
    q, k, v = torch.where(sel, qg, qu), torch.where(sel, kg, ku), vu
    o = attention(q, k, v, mask, cfg.head_dim ** -0.5).reshape(x.shape[0], -1)
    x = x + _branch(o, p[s + "wo"], is_gen_row, F.linear)
    h = torch.where(is_gen_row[:, None], rmsnorm(x, p[s + "ffn_norm"][GEN], eps),
                    rmsnorm(x, p[s + "ffn_norm"][UND], eps))
    if not cfg.is_moe:
        Fd = cfg.ffn_size

        def ffn(hh, w13, w2):
            gu = F.linear(hh, w13)
            return F.linear(F.silu(gu[:, :Fd]) * gu[:, Fd:], w2)

        y = torch.where(is_gen_row[:, None], ffn(h, p[s + "w13"][GEN], p[s + "w2"][GEN]),
                        ffn(h, p[s + "w13"][UND], p[s + "w2"][UND]))
    else:
        yu, lu = moe_ffn(h, p[s + "moe_und.gate"], p[s + "moe_und.w13"], p[s + "moe_und.w2"],
                         cfg.num_experts_per_tok, cfg.norm_topk_prob)
        yg, lg = moe_ffn(h, p[s + "moe_gen.gate"], p[s + "moe_gen.w13"], p[s + "moe_gen.w2"],
                         cfg.gen_num_experts_per_tok, cfg.norm_topk_prob)
        y = torch.where(is_gen_row[:, None], yg, yu)
        if aux is not None:
            aux.append((lu, lg))
    return x + y


def rope2d(x, px, py, theta):
    """Interleaved-pair 2-D rotary: first half of channels by column, second by row."""
    C = x.shape[-1]
    half = C // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, 2, dtype=torch.float32, device=x.device) / half))

    def rot(part, pos):
        ang = pos.float()[:, None] * inv[None, :]
        c, s = ang.cos(), ang.sin()
        x1, x2 = part[..., 0::2], part[..., 1::2]
        out = torch.empty_like(part)
        out[..., 0::2] = x1 * c - x2 * s
        out[..., 1::2] = x1 * s + x2 * c
        return out

    xf = x.float()
    return torch.cat([rot(xf[..., :half], px), rot(xf[..., half:], py)], dim=-1).to(x.dtype)


def vision_embed(p, br: str, patches, px, py, cfg: ModelConfig):
    """Block-major patches [T*m*m, patch_dim] -> token embeddings [T, hidden]."""
    w = p[f"vision_{br}.patch_w"]
    h = F.gelu(F.linear(patches.to(w.dtype), w, p[f"vision_{br}.patch_b"]))
    h = rope2d(h, px, py, cfg.rope_theta_vision)
    m2 = cfg.merge_size ** 2
    h = h.reshape(h.shape[0] // m2, m2 * h.shape[1])
    return F.linear(h, p[f"vision_{br}.merge_w"], p[f"vision_{br}.merge_b"])


def sinusoid(t, dim, max_period=10000.0):
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t[:, None].float() * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


def scalar_embed(p, name, t, cfg: ModelConfig):
    w1 = p[name + ".w1"]
    h = F.silu(F.linear(sinusoid(t, cfg.timestep_freq_dim).to(w1.dtype), w1, p[name + ".b1"]))
    return F.linear(h, p[name + ".w2"], p[name + ".b2"])


def fm_head(p, h, cfg: Optional[ModelConfig] = None, grids=None):
    """Generation head on the hidden states of image tokens ``h`` [T,H] -> predicted clean pixels
    [T, token_dim] in (row, column, channel) order.  MLP head, or (``cfg.use_pixel_head``) the
    convolutional decoder, which needs the token grid (rows, cols) of every image in ``grids``
    (tokens of one image are contiguous and in raster order)."""
    if cfg is None or not cfg.use_pixel_head:
        return F.linear(F.gelu(F.linear(h, p["fm_head.w1"], p["fm_head.b1"])), p["fm_head.w2"], p["fm_head.b2"])
    return pixel_head(p, h, grids, cfg)


def pixel_head(p, h, grids, cfg: ModelConfig):
    """ConvDecoder: [1,H,th,tw] -> pixel-shuffle(2) -> conv3x3 + GELU -> pixel-shuffle(2) -> conv3x3 ->
    pixel-shuffle(token_pixels / 4) -> [1,3,th*tp,tw*tp], regrouped into per-token pixel blocks
    (training/sensenovavl/model/modules/fm_modules.py:44-61; use in the training model
    modeling_sensenovavl_chat_mot.py:1410-1441)."""
    tp = cfg.token_pixels
    out, start = [], 0
    for th, tw in grids:
        n = th * tw
        x = h[start:start + n].view(1, th, tw, -1).permute(0, 3, 1, 2)
        start += n
        x = F.gelu(F.conv2d(F.pixel_shuffle(x, 2), p["fm_head.conv1_w"], p["fm_head.conv1_b"], padding=1))
        x = F.conv2d(F.pixel_shuffle(x, 2), p["fm_head.conv2_w"], p["fm_head.conv2_b"], padding=1)
        x = F.pixel_shuffle(x, tp // 4)                                     # [1,3,th*tp,tw*tp]
        x = x.view(3, th, tp, tw, tp).permute(1, 3, 2, 4, 0)                # (th, tw, p, q, c)
        out.append(x.reshape(n, tp * tp * 3))
    return torch.cat(out, dim=0)


def gen_image_grids(batch: PackedBatch):
    """(rows, cols) of every generation image of a packed batch, in the order of ``gen_rows``."""
    rows = batch.gen_rows
    if rows.numel() == 0:
        return []
    img = batch.meta[rows, 2]
    hh, ww = batch.pos3[1, rows], batch.pos3[2, rows]
    grids = []
    change = torch.nonzero(img[1:] != img[:-1]).flatten() + 1
    bounds = [0] + change.tolist() + [int(rows.numel())]
    for a, b in zip(bounds[:-1], bounds[1:]):
        grids.append((int(hh[a:b].max()) + 1, int(ww[a:b].max()) + 1))
    return grids


def embed_inputs(p, batch: PackedBatch, cfg: ModelConfig, noise16: Optional[torch.Tensor]):
    """Returns (x0 [S,H], z_tok, v_tok) — token embeddings with image rows filled in, and
    the flow-matching state / velocity targets in token pixel layout."""
    E = p["embed_tokens"]
    x = torch.zeros(batch.S, cfg.hidden_size, dtype=E.dtype, device=E.device)
    if batch.text_rows.numel():
        x = x.index_copy(0, batch.text_rows, E[batch.ids[batch.text_rows].long()])
    if batch.und_rows.numel():
        x = x.index_copy(0, batch.und_rows, vision_embed(p, "und", batch.und_patches, batch.und_px,
                                                         batch.und_py, cfg))
    z_tok = v_tok = None
    if batch.gen_rows.numel():
        m2 = cfg.merge_size ** 2
        t16 = batch.gen_t.repeat_interleave(m2)[:, None]
        ns16 = batch.gen_ns.repeat_interleave(m2)[:, None]
        z16 = t16 * batch.gen_x16 + (1 - t16) * noise16 * ns16
        emb = vision_embed(p, "gen", z16, batch.gen_px, batch.gen_py, cfg)
        emb = emb + scalar_embed(p, "timestep_embedder", batch.gen_t, cfg)
        if cfg.add_noise_scale_embedding:
            emb = emb + scalar_embed(p, "noise_scale_embedder", batch.gen_ns / cfg.noise_scale_max_value, cfg)
        x = x.index_copy(0, batch.gen_rows, emb.to(x.dtype))
        x_tok = patches_to_tokens(batch.gen_x16, cfg.patch_size, cfg.merge_size)
        z_tok = patches_to_tokens(z16, cfg.patch_size, cfg.merge_size)
        v_tok = (x_tok - z_tok) / (1 - batch.gen_t[:, None]).clamp_min(cfg.t_eps)
    return x, z_tok, v_tok


def training_loss(p: Dict[str, torch.Tensor], batch: PackedBatch, cfg: ModelConfig,
                  noise16: Optional[torch.Tensor] = None, ce_norm: Optional[float] = None,
                  gen_norm: Optional[float] = None):
    """Total SFT loss = ce_loss_weight * CE(text) + image_gen_loss_weight * FM MSE (+ MoE aux).
    ``ce_norm`` / ``gen_norm`` are the data-parallel averages of the weight sums (default:
    this batch's own sums).  Returns (loss, dict of parts)."""
    is_gen_row = batch.kind == KIND_GEN_IMG
    # padding rows of the generation partition also run through the generation weights
    row_group = batch.tile_group.repeat_interleave(128)
    is_gen_row = is_gen_row | (row_group == 1)
    x, z_tok, v_tok = embed_inputs(p, batch, cfg, noise16)
    mask = dense_mask(batch.meta, batch.meta)
    aux = [] if cfg.is_moe else None
    for l in range(cfg.num_layers):
        x = decoder_layer(p, l, x, is_gen_row, batch.pos3, mask, cfg, aux)
    total, parts = head_losses(p, x, batch, cfg, noise16, ce_norm, gen_norm, z_tok, v_tok, is_gen_row)
    if cfg.num_mtp_layers > 0:
        lm = mtp_loss(p, x, batch, cfg, is_gen_row, mask, ce_norm, aux)
        parts["mtp"] = lm.detach()
        total = total + cfg.mtp_loss_coeff * cfg.ce_loss_weight * lm
    if aux:
        la = x.new_zeros((), dtype=torch.float32)
        lz = x.new_zeros((), dtype=torch.float32)
        split = cfg.moe_balance_image_ratio > 0 or cfg.moe_balance_text_ratio > 0
        for lu, lg in aux:
            real = batch.kind != 0                          # padding rows do not count
            und, gen = ~is_gen_row & real, is_gen_row & real
            if gen.any():
                la = la + cfg.moe_balance_gen_ratio * load_balance_loss(lg[gen], cfg.gen_num_experts_per_tok)
            if und.any():
                if split:
                    # image and text tokens of the understanding branch balanced separately
                    # (training/sensenovalm/model/modeling_qwen3_moe_mot.py:824-920)
                    img = und & (batch.kind == 2)
                    txt = und & (batch.kind != 2)
                    for rows, ratio in ((txt, cfg.moe_balance_text_ratio), (img, cfg.moe_balance_image_ratio)):
                        if rows.any():
                            la = la + cfg.moe_balance_und_ratio * ratio * load_balance_loss(lu[rows], cfg.num_experts_per_tok)
                else:
                    la = la + cfg.moe_balance_und_ratio * load_balance_loss(lu[und], cfg.num_experts_per_tok)
            if cfg.router_z_loss_coef > 0:
                for lg_, rows in ((lu, und), (lg, gen)):
                    if rows.any():
                        lz = lz + torch.logsumexp(lg_[rows].float(), dim=-1).pow(2).mean()
        parts["moe_aux"] = la.detach()
        total = total + cfg.router_aux_loss_coef * la
        if cfg.router_z_loss_coef > 0:
            parts["moe_z_loss"] = lz.detach()
            total = total + cfg.router_z_loss_coef * lz
    return total, parts


def mtp_shift(batch: PackedBatch, k: int):
    """Rows r whose next k rows are text of the same document, laid out contiguously: returns
    (valid [S] bool, index of row r + k clipped to the batch)."""
    S = batch.ids.numel()
    idx = torch.arange(S, device=batch.ids.device)
    tgt = (idx + k).clamp_max(S - 1)
    doc = batch.meta[:, 0]
    pos = batch.meta[:, 1]
    text = batch.kind == 1
    ok = (idx + k < S) & text & text[tgt] & (doc[tgt] == doc) & (pos[tgt] == pos + k)
    return ok, tgt


def mtp_loss(p, x, batch: PackedBatch, cfg: ModelConfig, is_gen_row, mask, ce_norm=None, aux=None):
    """Multi-token prediction (training/sensenovalm/model/mtp.py:58-108, loss assembly
    core/scheduler/no_pipeline_scheduler.py:174-190): head k takes the hidden state of the previous
    depth and the embedding of the token k + 1 positions ahead, runs one more decoder layer and
    predicts, through the shared final norm and LM head, the label k + 1 positions ahead of the
    main one.  Only text rows whose lookahead stays inside the same run of text are used."""
    eps = cfg.rms_eps
    total = x.new_zeros((), dtype=torch.float32)
    h = x
    norm = ce_norm if ce_norm is not None else max(batch.ce_weight_sum, 1e-12)
    for k in range(cfg.num_mtp_layers):
        ok, tgt = mtp_shift(batch, k + 1)
        emb = F.embedding(batch.ids[tgt].long(), p["embed_tokens"])
        emb = torch.where(ok[:, None], emb, torch.zeros_like(emb))
        z = torch.cat([rmsnorm(h, p[f"mtp.{k}.norm_hidden"], eps), rmsnorm(emb, p[f"mtp.{k}.norm_embed"], eps)], dim=1)
        h = decoder_layer(p, f"mtp.{k}.layer.", F.linear(z, p[f"mtp.{k}.proj"]), is_gen_row, batch.pos3, mask, cfg, aux)
        rows = (ok & (batch.labels[tgt] >= 0) & (batch.loss_w[tgt] > 0)).nonzero().flatten()
        if rows.numel():
            hf = rmsnorm(h[rows], p["final_norm"][UND], eps)
            logits = F.linear(hf, p["lm_head"]).float()
            t = tgt[rows]
            ce_rows = F.cross_entropy(logits, batch.labels[t].long(), reduction="none")
            total = total + (ce_rows * batch.loss_w[t]).sum() / norm
    return total


def head_losses(p, x, batch: PackedBatch, cfg: ModelConfig, noise16=None, ce_norm=None, gen_norm=None,
                z_tok=None, v_tok=None, is_gen_row=None):
    """Final norm, LM head CE and flow-matching loss on the last hidden state ``x`` [S,H]."""
    if is_gen_row is None:
        is_gen_row = (batch.kind == KIND_GEN_IMG) | (batch.tile_group.repeat_interleave(128) == 1)
    if z_tok is None and batch.gen_rows.numel():
        m2 = cfg.merge_size ** 2
        t16 = batch.gen_t.repeat_interleave(m2)[:, None]
        ns16 = batch.gen_ns.repeat_interleave(m2)[:, None]
        z16 = t16 * batch.gen_x16 + (1 - t16) * noise16 * ns16
        x_tok = patches_to_tokens(batch.gen_x16, cfg.patch_size, cfg.merge_size)
        z_tok = patches_to_tokens(z16, cfg.patch_size, cfg.merge_size)
        v_tok = (x_tok - z_tok) / (1 - batch.gen_t[:, None]).clamp_min(cfg.t_eps)
    eps = cfg.rms_eps
    h = torch.where(is_gen_row[:, None], rmsnorm(x, p["final_norm"][GEN], eps),
                    rmsnorm(x, p["final_norm"][UND], eps))
    parts = {}
    total = x.new_zeros((), dtype=torch.float32)
    if batch.label_rows.numel():
        logits = F.linear(h[batch.label_rows], p["lm_head"]).float()
        tgt = batch.labels[batch.label_rows].long()
        w = batch.loss_w[batch.label_rows]
        ce_rows = F.cross_entropy(logits, tgt, reduction="none")
        norm = ce_norm if ce_norm is not None else max(batch.ce_weight_sum, 1e-12)
        ce = (ce_rows * w).sum() / norm
        parts["ce"] = ce.detach()
        total = total + cfg.ce_loss_weight * ce
    if batch.gen_rows.numel():
        x_pred = fm_head(p, h[batch.gen_rows], cfg, gen_image_grids(batch) if cfg.use_pixel_head else None).float()
        den = (1 - batch.gen_t[:, None]).clamp_min(cfg.t_eps)
        v_pred = (x_pred - z_tok) / den
        row = ((v_pred - v_tok) ** 2).mean(dim=1)
        norm = gen_norm if gen_norm is not None else max(batch.gen_weight_sum, 1.0)
        fm = (row * batch.gen_w).sum() / norm
        parts["fm"] = fm.detach()
        total = total + cfg.image_gen_loss_weight * fm
    return total, parts


def load_balance_loss(logits, top_k):
    """E * sum_i f_i P_i with f the fraction of routed slots and P the mean gate probability
    (training/sensenovalm/model/modeling_qwen3_moe_mot.py:754-969, unweighted form)."""
    probs = torch.softmax(logits.float(), dim=-1)
    E = probs.shape[-1]
    _, ti = torch.topk(probs, top_k, dim=-1)
    f = F.one_hot(ti, E).float().sum(1).mean(0) / top_k
    return E * (f * probs.mean(0)).sum()


# ---------------------------------------------------------------------------
# inference oracle (no cache: the whole [prompt | image] sequence is recomputed)
# ---------------------------------------------------------------------------
def t2i_reference(p, cfg: ModelConfig, cond_ids, uncond_ids, image_size, num_steps, cfg_scale,
                  timestep_shift, noise, cfg_norm="none", t_eps=0.02):
    """Text-to-image sampling in plain PyTorch, batch 1 (modeling_neo_chat.py:1691-1860)."""
    from ..data.batch import apply_time_schedule, patchify_block_major, tokens_to_patches
    from ..ops.attention import make_meta
    dev = p["embed_tokens"].device
    W, Hh = image_size
    tp = cfg.token_pixels
    th, tw = Hh // tp, W // tp
    T = th * tw
    ns = min(math.sqrt(T / float(cfg.noise_scale_base_image_seq_len)) * cfg.noise_scale
             if cfg.noise_scale_mode in ("resolution", "dynamic") else cfg.noise_scale, cfg.noise_scale_max_value)
    img = ns * noise.float()[0]
    p16, px, py, _, _ = patchify_block_major(img.cpu(), cfg.patch_size, cfg.merge_size)
    px, py = px.to(dev), py.to(dev)
    z = patches_to_tokens(p16.to(dev), cfg.patch_size, cfg.merge_size)
    ts = apply_time_schedule(torch.linspace(0, 1, num_steps + 1), T, cfg, timestep_shift=timestep_shift).tolist()
    hh = torch.arange(th).view(th, 1).expand(th, tw).reshape(-1).to(dev)
    ww = torch.arange(tw).view(1, tw).expand(th, tw).reshape(-1).to(dev)

    def predict(ids, z, t):
        n = ids.numel()
        S = n + T
        x_txt = p["embed_tokens"][ids.to(dev).long()]
        emb = vision_embed(p, "gen", tokens_to_patches(z, cfg.patch_size, cfg.merge_size), px, py, cfg)
        tt = torch.full((T,), t, device=dev)
        emb = emb + scalar_embed(p, "timestep_embedder", tt, cfg)
        if cfg.add_noise_scale_embedding:
            emb = emb + scalar_embed(p, "noise_scale_embedder", torch.full((T,), ns / cfg.noise_scale_max_value, device=dev), cfg)
        x = torch.cat([x_txt, emb.to(x_txt.dtype)])
        is_gen = torch.cat([torch.zeros(n, dtype=torch.bool), torch.ones(T, dtype=torch.bool)]).to(dev)
        pos = torch.cat([torch.arange(n), torch.full((T,), n)]).to(dev)
        pos3 = torch.stack([pos, torch.cat([torch.zeros(n, dtype=torch.long, device=dev), hh]),
                            torch.cat([torch.zeros(n, dtype=torch.long, device=dev), ww])])
        imgid = torch.cat([torch.zeros(n), torch.ones(T)]).to(dev)
        meta = make_meta(torch.zeros(S, device=dev), pos, imgid, is_gen)
        mask = dense_mask(meta, meta)
        for l in range(cfg.num_layers):
            x = decoder_layer(p, l, x, is_gen, pos3, mask, cfg)
        h = rmsnorm(x[n:], p["final_norm"][GEN], cfg.rms_eps)
        x_pred = fm_head(p, h, cfg, [(th, tw)]).float()
        return (x_pred - z) / max(1 - t, t_eps)

    for i in range(num_steps):
        t, t_next = ts[i], ts[i + 1]
        vc = predict(cond_ids, z, t)
        if cfg_scale > 1 and uncond_ids is not None:
            vu = predict(uncond_ids, z, t)
            v = vu + cfg_scale * (vc - vu)
            if cfg_norm == "global":
                v = v * (vc.norm() / (v.norm() + 1e-8)).clamp(max=1.0)
            elif cfg_norm == "channel":
                v = v * (vc.norm(dim=-1, keepdim=True) / (v.norm(dim=-1, keepdim=True) + 1e-8)).clamp(max=1.0)
            elif cfg_norm == "cfg_zero_star":
                a = (vc * vu).sum() / (vu.pow(2).sum() + 1e-8)
                v = vc * 0 if i == 0 else vu * a + cfg_scale * (vc - vu * a)
        else:
            v = vc
        z = z + (t_next - t) * v
    return z.reshape(th, tw, tp, tp, 3).permute(4, 0, 2, 1, 3).reshape(1, 3, Hh, W)
