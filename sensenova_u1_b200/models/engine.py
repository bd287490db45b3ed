"""CUDA training engine of the dense NEO-unify MoT model: an explicit forward and
backward pass over hand-written sm_100a kernels.

There is no autograd graph on this path.  The forward pass keeps only the input
of every decoder layer; the backward pass recomputes a layer's activations from
that input and then walks it backwards (the reference checkpoints every layer as
well, ``checkpoint=1``, training/sensenovalm/model/modeling_qwen3_moe_mot.py:299).
Weight gradients are accumulated by the GEMM epilogue straight into the flat
gradient arena, the losses produce their own gradients in the same kernel that
evaluates them, and every buffer comes from a fixed workspace, so a step makes
no allocation and no host synchronisation.

Row layout: ``[generation rows | understanding rows]`` with 128-row tiles owned
by one branch (see ``data/batch.py``); every projection is ONE grouped GEMM
launch with a per-tile weight-set index, replacing the slice / cat routing of
the reference (modeling_qwen3_moe_mot.py:323-369).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..config import ModelConfig
from ..data.batch import KIND_TEXT, PackedBatch, patches_to_tokens
from ..ops import attention as attn_ops
from ..ops import fused, gemm
from ..ops.gemm import OUT_BF16_ACC, OUT_BF16_STORE
from . import oracle
from .params import ParamStore


class Workspace:
    """Named, shape-keyed scratch buffers that live as long as the engine."""

    def __init__(self, device):
        self.device = device
        self.bufs: Dict[str, torch.Tensor] = {}

    def get(self, name, shape, dtype=torch.bfloat16, zero=False):
        key = name
        t = self.bufs.get(key)
        n = 1
        for s in shape:
            n *= s
        if t is None or t.numel() < n or t.dtype != dtype:
            t = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
            self.bufs[key] = t
        out = t[:n].view(shape)
        if zero:
            out.zero_()
        return out

    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in self.bufs.values())


class MoTEngine:
    def __init__(self, cfg: ModelConfig, store: ParamStore):
        if cfg.head_dim != 128:
            raise ValueError("the sm_100a attention kernels need head_dim 128")
        if cfg.is_moe and type(self) is MoTEngine:
            raise ValueError("MoTEngine covers the dense model; use MoEMoTEngine for expert layers")
        self.cfg = cfg
        self.store = store
        self.p, self.g = store.p, store.g
        self.dev = store.device
        self.ws = Workspace(self.dev)
        inv_t, inv_hw = oracle.rope_inv_freq(cfg, self.dev)
        self.inv_t, self.inv_hw = inv_t.contiguous(), inv_hw.contiguous()
        half = cfg.vision_hidden // 2
        self.inv_v = (1.0 / (cfg.rope_theta_vision ** (
            torch.arange(0, half, 2, dtype=torch.float32, device=self.dev) / half))).contiguous()
        self.loss_acc = torch.zeros(12, dtype=torch.float32, device=self.dev)  # [0:4] CE, [4] FM, [8:12] MTP CE
        self.scale = cfg.head_dim ** -0.5
        # per-task generation losses for the log (record_metrics.py:463-467 of the reference): two small index_adds
        self.per_task_losses = False
        self.task_acc = torch.zeros(2, 8, dtype=torch.float32, device=self.dev)
        self.ce_chunk = 2048
        # Activation policy.  "full": keep only each layer's input and recompute the layer in backward
        # (fits one 180 GB GPU).  "attention": also keep the attention output and log-sum-exp, so the
        # attention forward is not repeated.  "none": keep the projections too; backward recomputes only
        # the cheap element-wise pieces.  "auto" picks by free memory at the first step.
        self.recompute = "auto"
        self._mode, self._mode_S = None, 0
        # parallel.context_attention.ContextParallelAttention: one packed sequence split over ranks
        self.cp = None
        # MoT branches (0 understanding, 1 generation) whose decoder weights are frozen: the grouped
        # weight-gradient GEMMs skip them (the trainer clears whatever gradient is left)
        self.skip_wgrad_groups = ()
        # callbacks for communication overlap: bucket names 'front', 'layer.<i>', 'head'
        self.on_grads_ready = None
        self.on_weights_needed = None
        # weight-parallel mode: called when the backward pass of a micro-batch starts, and before the backward of
        # every decoder layer (the layer's full weights are gathered, its gradient staging slot is cleared)
        self.on_backward_begin = None
        self.on_layer_backward_begin = None
        # tensor parallel (parallel/tensor_engine.py): this engine then runs the local slice of every projection
        # (``cfg`` is the local configuration) and completes the four partial sums per layer with ``tp.all_reduce_``
        self.tp = None

    @staticmethod
    def _pfx(l) -> str:
        """Parameter prefix of a decoder layer: an index of the main stack, or the full prefix of an extra
        layer (the decoder layers of the multi-token-prediction heads)."""
        return l if isinstance(l, str) else f"layers.{l}."

    def _tp_sum(self, t):
        """Completes a partial sum over the tensor-parallel group (no-op without tensor parallelism)."""
        if self.tp is not None:
            self.tp.all_reduce_(t)
        return t

    def _res(self, x):
        """The residual operand of a row-parallel product: added once, by tensor-parallel rank 0."""
        return x if (self.tp is None or self.tp.rank == 0) else None

    def _need(self, bucket):
        if self.on_weights_needed is not None:
            self.on_weights_needed(bucket)

    def _ready(self, bucket):
        if self.on_grads_ready is not None:
            self.on_grads_ready(bucket)

    # ------------------------------------------------------------------ utils
    def _linear(self, x, w, b=None, out=None):
        return gemm.gemm_nt(x, w, out=out, residual=b)

    def _wgrad(self, dy, x, name):
        gemm.gemm_tn(dy, x, out=self.g[name], out_mode=OUT_BF16_ACC)

    def _bgrad(self, dy, name):
        fused.colsum(dy, self.g[name])

    # --------------------------------------------------------------- vision
    def _vision_fwd(self, br, patches, px, py, tag):
        cfg, ws = self.cfg, self.ws
        P_, Cv = patches.shape[0], cfg.vision_hidden
        m2 = cfg.merge_size ** 2
        a1 = self._linear(patches, self.p[f"vision_{br}.patch_w"], self.p[f"vision_{br}.patch_b"],
                          out=ws.get(tag + ".a1", (P_, Cv)))
        g1 = fused.gelu_fwd(a1, ws.get(tag + ".g1", (P_, Cv)))
        r1 = fused.rope2d(g1, ws.get(tag + ".r1", (P_, Cv)), px, py, self.inv_v)
        emb = self._linear(r1.view(P_ // m2, m2 * Cv), self.p[f"vision_{br}.merge_w"],
                           self.p[f"vision_{br}.merge_b"], out=ws.get(tag + ".emb", (P_ // m2, cfg.hidden_size)))
        return emb, (patches, a1, r1, px, py)

    def _vision_bwd(self, br, d_emb, saved, tag):
        cfg, ws = self.cfg, self.ws
        patches, a1, r1, px, py = saved
        P_, Cv = a1.shape
        m2 = cfg.merge_size ** 2
        r1v = r1.view(P_ // m2, m2 * Cv)
        self._wgrad(d_emb, r1v, f"vision_{br}.merge_w")
        self._bgrad(d_emb, f"vision_{br}.merge_b")
        d_r1 = gemm.gemm_nn(d_emb, self.p[f"vision_{br}.merge_w"], out=ws.get(tag + ".d_r1", (P_ // m2, m2 * Cv)))
        d_g1 = fused.rope2d(d_r1.view(P_, Cv), ws.get(tag + ".d_g1", (P_, Cv)), px, py, self.inv_v, inverse=True)
        d_a1 = fused.gelu_bwd(a1, d_g1, d_g1)
        self._wgrad(d_a1, patches, f"vision_{br}.patch_w")
        self._bgrad(d_a1, f"vision_{br}.patch_b")

    # ----------------------------------------------------- convolutional pixel head
    def _conv_weights(self):
        """The two 3x3 kernels as GEMM operands [O, 3*3*C] (tap-major columns, matching ``ps_im2col``)."""
        p = self.p
        w1, w2 = p["fm_head.conv1_w"], p["fm_head.conv2_w"]
        return (w1.permute(0, 2, 3, 1).reshape(w1.shape[0], -1).contiguous(),
                w2.permute(0, 2, 3, 1).reshape(w2.shape[0], -1).contiguous())

    def _pixel_head_fwd(self, h_gen, grids, x_pred):
        """ConvDecoder on the generation tokens (image by image: tokens of an image are contiguous, in raster order):
        pixel-shuffle + conv3x3 as patch gather + GEMM, GELU, again, then the last pixel shuffle straight into the
        per-token pixel blocks ``x_pred`` [Tg, token_dim].  Returns what the backward needs."""
        cfg, ws = self.cfg, self.ws
        H, O1, r = cfg.hidden_size, cfg.pixel_head_dim, cfg.token_pixels // 4
        W1p, W2p = self._conv_weights()
        saved, a = [], 0
        for i, (gh, gw) in enumerate(grids):
            n = gh * gw
            x = h_gen[a:a + n]
            A1 = fused.ps_im2col(x, ws.get(f"ph{i}.A1", (4 * n, 9 * H // 4)), gh, gw, H // 4)
            c1 = gemm.gemm_nt(A1, W1p, out=ws.get(f"ph{i}.c1", (4 * n, O1)), residual=self.p["fm_head.conv1_b"])
            g1 = fused.gelu_fwd(c1, ws.get(f"ph{i}.g1", (4 * n, O1)))
            A2 = fused.ps_im2col(g1, ws.get(f"ph{i}.A2", (16 * n, 9 * O1 // 4)), 2 * gh, 2 * gw, O1 // 4)
            y2 = gemm.gemm_nt(A2, W2p, out=ws.get(f"ph{i}.y2", (16 * n, 3 * r * r)), residual=self.p["fm_head.conv2_b"])
            fused.pixel_regroup(y2, x_pred[a:a + n], gh, gw, r)
            saved.append((a, n, gh, gw, A1, c1, g1, A2))
            a += n
        return dict(saved=saved, W1p=W1p, W2p=W2p)

    def _pixel_head_bwd(self, d_xp, st, d_hgen):
        """Backward of :meth:`_pixel_head_fwd`: weight / bias gradients into the arena, d loss / d h_gen."""
        cfg, ws, g = self.cfg, self.ws, self.g
        H, O1, r = cfg.hidden_size, cfg.pixel_head_dim, cfg.token_pixels // 4
        W1p, W2p = st["W1p"], st["W2p"]
        dW1p = ws.get("ph.dW1p", tuple(W1p.shape), zero=True)
        dW2p = ws.get("ph.dW2p", tuple(W2p.shape), zero=True)
        for i, (a, n, gh, gw, A1, c1, g1, A2) in enumerate(st["saved"]):
            d_y2 = fused.pixel_regroup(ws.get(f"ph{i}.dy2", (16 * n, 3 * r * r)), d_xp[a:a + n], gh, gw, r, to_y=True)
            gemm.gemm_tn(d_y2, A2, out=dW2p, out_mode=OUT_BF16_ACC)
            self._bgrad(d_y2, "fm_head.conv2_b")
            dA2 = gemm.gemm_nn(d_y2, W2p, out=ws.get(f"ph{i}.A2", (16 * n, 9 * O1 // 4)))       # A2 is dead now
            d_g1 = fused.ps_col2im(dA2, ws.get(f"ph{i}.g1", (4 * n, O1)), 2 * gh, 2 * gw, O1 // 4)
            d_c1 = fused.gelu_bwd(c1, d_g1, d_g1)
            gemm.gemm_tn(d_c1, A1, out=dW1p, out_mode=OUT_BF16_ACC)
            self._bgrad(d_c1, "fm_head.conv1_b")
            dA1 = gemm.gemm_nn(d_c1, W1p, out=ws.get(f"ph{i}.A1", (4 * n, 9 * H // 4)))
            fused.ps_col2im(dA1, d_hgen[a:a + n], gh, gw, H // 4)
        w1, w2 = g["fm_head.conv1_w"], g["fm_head.conv2_w"]
        w1.add_(dW1p.view(w1.shape[0], 3, 3, w1.shape[1]).permute(0, 3, 1, 2))
        w2.add_(dW2p.view(w2.shape[0], 3, 3, w2.shape[1]).permute(0, 3, 1, 2))

    def _scalar_embed_fwd(self, name, t, tag):
        cfg, ws = self.cfg, self.ws
        s = oracle.sinusoid(t, cfg.timestep_freq_dim).to(torch.bfloat16)
        a = self._linear(s, self.p[name + ".w1"], self.p[name + ".b1"], out=ws.get(tag + ".a", (t.numel(), cfg.hidden_size)))
        h = torch.nn.functional.silu(a)
        e = self._linear(h, self.p[name + ".w2"], self.p[name + ".b2"], out=ws.get(tag + ".e", (t.numel(), cfg.hidden_size)))
        return e, (s, a, h)

    def _scalar_embed_bwd(self, name, d_e, saved):
        s, a, h = saved
        self._wgrad(d_e, h, name + ".w2")
        self._bgrad(d_e, name + ".b2")
        d_h = gemm.gemm_nn(d_e, self.p[name + ".w2"])
        af = a.float()
        sg = torch.sigmoid(af)
        d_a = (d_h.float() * (sg * (1 + af * (1 - sg)))).to(torch.bfloat16)
        self._wgrad(d_a, s, name + ".w1")
        self._bgrad(d_a, name + ".b1")

    # ---------------------------------------------------------------- layer
    def _layer_fwd(self, l, x, out, b: PackedBatch, plan, keep=False):
        """out = layer_l(x).  With ``keep`` the intermediates stay in the workspace for backward."""
        cfg, ws, p = self.cfg, self.ws, self.p
        S, H = x.shape
        s = self._pfx(l)
        tg = b.tile_group
        qd, kd = cfg.q_dim, cfg.kv_dim
        QKV = qd + 2 * kd
        # buffers that the chosen activation policy keeps per layer get a per-layer name
        pa = f"L{l}." if self._mode in ("attention", "none") else ""      # attention output, lse
        pn = f"L{l}." if self._mode == "none" else ""                     # projections
        h1 = ws.get("h1", (S, H)); rstd1 = ws.get(pn + "rstd1", (S,), torch.float32)
        fused.rmsnorm_fwd(x, p[s + "attn_norm"], tg, h1, rstd1, cfg.rms_eps)
        qkv = gemm.gemm_nt(h1, p[s + "wqkv"], out=ws.get(pn + "qkv", (S, QKV)), tile_group=tg)
        qk = ws.get(pn + "qk", (S, qd + kd))
        fused.qknorm_rope_fwd(qkv, qk, p[s + "qk_norm"], tg, b.pos3, self.inv_t, self.inv_hw,
                              cfg.num_heads, cfg.num_kv_heads, cfg.rms_eps)
        q = qk[:, :qd].unflatten(1, (cfg.num_heads, 128))
        k = qk[:, qd:].unflatten(1, (cfg.num_kv_heads, 128))
        v = qkv[:, qd + kd:].unflatten(1, (cfg.num_kv_heads, 128))
        o = ws.get(pa + "attn_o", (S, cfg.num_heads, 128))
        lse_buf = ws.get(pa + "lse", (cfg.num_heads, S), torch.float32)
        if keep and self._mode == "attention":
            lse = lse_buf                      # kept from the forward pass: no second attention forward
        elif self.cp is not None:
            # context parallel: my K/V go to symmetric memory, attention walks every rank's key block
            self.cp.publish(k, v)
            o, lse = self.cp.forward(q, self.scale, out=o, lse=lse_buf)
        else:
            o, lse = attn_ops.attention_fwd(q, k, v, plan, self.scale, out=o, lse=lse_buf)
        x1 = self._tp_sum(gemm.gemm_nt(o.view(S, qd), p[s + "wo"], out=ws.get(pn + "x1", (S, H)), tile_group=tg,
                                       residual=self._res(x)))
        h2 = ws.get("h2", (S, H)); rstd2 = ws.get(pn + "rstd2", (S,), torch.float32)
        fused.rmsnorm_fwd(x1, p[s + "ffn_norm"], tg, h2, rstd2, cfg.rms_eps)
        ffn = self._ffn_fwd(l, h2, x1, out, b, pn)
        if keep:
            a = dict(h1=h1, rstd1=rstd1, qkv=qkv, qk=qk, q=q, k=k, v=v, o=o, lse=lse, x1=x1, h2=h2, rstd2=rstd2)
            a.update(ffn)
            return a
        return None

    def _ffn_fwd(self, l, h2, x1, out, b: PackedBatch, pn: str = ""):
        """out = x1 + FFN(h2) (skipped when out is None); returns what the backward needs."""
        cfg, ws, p = self.cfg, self.ws, self.p
        s = self._pfx(l)
        S = h2.shape[0]
        tg = b.tile_group
        gu = gemm.gemm_nt(h2, p[s + "w13"], out=ws.get(pn + "gu", (S, 2 * cfg.ffn_size)), tile_group=tg)
        act = fused.swiglu_fwd(gu, ws.get("act", (S, cfg.ffn_size)))
        if out is not None:
            self._tp_sum(gemm.gemm_nt(act, p[s + "w2"], out=out, tile_group=tg, residual=self._res(x1)))
        return dict(gu=gu, act=act)

    def _saved(self, l, x, b: PackedBatch):
        """Intermediates of layer l from the buffers the forward pass kept ("none" policy); only the
        two RMSNorms and the SwiGLU are evaluated again."""
        cfg, ws, p = self.cfg, self.ws, self.p
        S, H = x.shape
        s, pn, tg = self._pfx(l), f"L{l}.", b.tile_group
        qd, kd = cfg.q_dim, cfg.kv_dim
        rstd1, rstd2 = ws.get(pn + "rstd1", (S,), torch.float32), ws.get(pn + "rstd2", (S,), torch.float32)
        h1 = fused.rmsnorm_fwd(x, p[s + "attn_norm"], tg, ws.get("h1", (S, H)), rstd1, cfg.rms_eps)
        qkv, qk = ws.get(pn + "qkv", (S, qd + 2 * kd)), ws.get(pn + "qk", (S, qd + kd))
        x1 = ws.get(pn + "x1", (S, H))
        h2 = fused.rmsnorm_fwd(x1, p[s + "ffn_norm"], tg, ws.get("h2", (S, H)), rstd2, cfg.rms_eps)
        gu = ws.get(pn + "gu", (S, 2 * cfg.ffn_size))
        act = fused.swiglu_fwd(gu, ws.get("act", (S, cfg.ffn_size)))
        return dict(h1=h1, rstd1=rstd1, qkv=qkv, qk=qk, q=qk[:, :qd].unflatten(1, (cfg.num_heads, 128)),
                    k=qk[:, qd:].unflatten(1, (cfg.num_kv_heads, 128)),
                    v=qkv[:, qd + kd:].unflatten(1, (cfg.num_kv_heads, 128)),
                    o=ws.get(pn + "attn_o", (S, cfg.num_heads, 128)),
                    lse=ws.get(pn + "lse", (cfg.num_heads, S), torch.float32), x1=x1, h2=h2, rstd2=rstd2, gu=gu, act=act)

    def _pick_mode(self, S: int) -> str:
        if self.recompute != "auto":
            return self.recompute
        if self.cfg.is_moe or self.dev.type != "cuda":
            return "full"
        cfg = self.cfg
        free, _ = torch.cuda.mem_get_info(self.dev)
        L = cfg.num_layers
        per_attn = S * cfg.q_dim * 2 + cfg.num_heads * S * 4
        per_none = per_attn + S * 2 * (cfg.q_dim + 2 * cfg.kv_dim + cfg.q_dim + cfg.kv_dim + cfg.hidden_size + 2 * cfg.ffn_size) + 8 * S
        shared = (L + 1) * S * cfg.hidden_size * 2 + 12 * S * max(2 * cfg.ffn_size, cfg.hidden_size) * 2 + (6 << 30)
        if free > shared + L * per_none:
            return "none"
        if free > shared + L * per_attn:
            return "attention"
        return "full"

    def _ffn_bwd(self, l, a, dy, b: PackedBatch):
        """Returns d loss / d h2 (FFN input after the norm); accumulates the FFN weight gradients."""
        cfg, ws, p, g = self.cfg, self.ws, self.p, self.g
        s = self._pfx(l)
        S, H = dy.shape
        tg, kb, ke = b.tile_group, self._kb, self._ke
        wmode = self._wgrad_mode(l)
        d_act = gemm.gemm_nn(dy, p[s + "w2"], out=ws.get("d_act", (S, cfg.ffn_size)), tile_group=tg)
        gemm.gemm_tn(dy, a["act"], out=g[s + "w2"], k_begin=kb, k_end=ke, num_groups=2, out_mode=wmode)
        d_gu = fused.swiglu_bwd(a["gu"], d_act, ws.get("d_gu", (S, 2 * cfg.ffn_size)))
        d_h2 = gemm.gemm_nn(d_gu, p[s + "w13"], out=ws.get("d_h", (S, H)), tile_group=tg)
        gemm.gemm_tn(d_gu, a["h2"], out=g[s + "w13"], k_begin=kb, k_end=ke, num_groups=2, out_mode=wmode)
        return self._tp_sum(d_h2)

    # set by the trainer for the first micro-batch of a step whose layer-matrix gradients were not cleared
    store_first = False

    def _wgrad_mode(self, l) -> int:
        """Output mode of the weight-gradient products of decoder layer ``l``: stored (not added) on the first
        micro-batch when the trainer skipped clearing them; MTP layers and every other tensor always add."""
        return OUT_BF16_STORE if (self.store_first and isinstance(l, int)) else OUT_BF16_ACC

    def _layer_bwd(self, l, x, dy, dx_out, b: PackedBatch, plan):
        """Recomputes layer l from its input x and writes d loss / d x into dx_out."""
        cfg, ws, p, g = self.cfg, self.ws, self.p, self.g
        S, H = x.shape
        s = self._pfx(l)
        tg = b.tile_group
        kb, ke = self._kb, self._ke
        qd, kd = cfg.q_dim, cfg.kv_dim
        a = self._saved(l, x, b) if self._mode == "none" else self._layer_fwd(l, x, None, b, plan, keep=True)
        d_h2 = self._ffn_bwd(l, a, dy, b)
        d_x1 = fused.rmsnorm_bwd(d_h2, a["x1"], p[s + "ffn_norm"], a["rstd2"], tg, dy,
                                 ws.get("d_x1", (S, H)), g[s + "ffn_norm"])
        # attention
        d_o = gemm.gemm_nn(d_x1, p[s + "wo"], out=ws.get("d_o", (S, qd)), tile_group=tg)
        gemm.gemm_tn(d_x1, a["o"].view(S, qd), out=g[s + "wo"], k_begin=kb, k_end=ke, num_groups=2,
                     out_mode=self._wgrad_mode(l))
        d_qkv = ws.get("d_qkv", (S, qd + 2 * kd))
        dq = d_qkv[:, :qd].unflatten(1, (cfg.num_heads, 128))
        dk = d_qkv[:, qd:qd + kd].unflatten(1, (cfg.num_kv_heads, 128))
        dv = d_qkv[:, qd + kd:].unflatten(1, (cfg.num_kv_heads, 128))
        if self.cp is not None:
            if self._mode != "full":           # K/V of this layer were not just re-published by a recompute
                self.cp.publish(a["k"], a["v"])
            self.cp.backward(a["q"], a["o"], d_o.view(S, cfg.num_heads, 128), a["lse"], self.scale,
                             dq=dq, dk=dk, dv=dv)
        else:
            attn_ops.attention_bwd(a["q"], a["k"], a["v"], a["o"], d_o.view(S, cfg.num_heads, 128), a["lse"],
                                   plan, self.scale, dq=dq, dk=dk, dv=dv,
                                   delta=ws.get("delta", (cfg.num_heads, S), torch.float32))
        fused.qknorm_rope_bwd(a["qkv"], d_qkv, p[s + "qk_norm"], g[s + "qk_norm"], tg, b.pos3,
                              self.inv_t, self.inv_hw, cfg.num_heads, cfg.num_kv_heads, cfg.rms_eps)
        d_h1 = gemm.gemm_nn(d_qkv, p[s + "wqkv"], out=ws.get("d_h", (S, H)), tile_group=tg)
        gemm.gemm_tn(d_qkv, a["h1"], out=g[s + "wqkv"], k_begin=kb, k_end=ke, num_groups=2,
                     out_mode=self._wgrad_mode(l))
        self._tp_sum(d_h1)
        fused.rmsnorm_bwd(d_h1, x, p[s + "attn_norm"], a["rstd1"], tg, d_x1, dx_out, g[s + "attn_norm"])

    # ----------------------------------------------------------------- step
    def forward_backward(self, b: PackedBatch, noise16: Optional[torch.Tensor] = None,
                         ce_norm: Optional[float] = None, gen_norm: Optional[float] = None,
                         loss_scale: float = 1.0, backward: bool = True):
        """One micro-batch.  Gradients are accumulated into ``store.grad_arena``.
        Returns device scalars {'loss', 'ce', 'fm', 'ce_correct', 'ce_rows'} (no sync)."""
        st = self.begin(b, noise16, ce_norm, gen_norm, loss_scale, backward)
        self.embed_fwd(st)
        self.layers_fwd(st)
        out = self.heads(st)
        if not backward:
            return out
        self.layers_bwd(st)
        self.embed_bwd(st)
        return out

    # The phases below are what ``forward_backward`` is made of.  A pipeline stage calls a subset of them per
    # micro-batch (parallel/pipeline_engine.py): the first stage ``embed_fwd`` + ``layers_fwd`` and later
    # ``layers_bwd`` + ``embed_bwd``, a middle stage only the layer phases, the last stage ``layers_fwd`` +
    # ``heads`` and later ``layers_bwd``.  ``slot`` names the set of activation buffers of a micro-batch, so that
    # several micro-batches can be in flight between their forward and backward phases.
    def begin(self, b: PackedBatch, noise16=None, ce_norm=None, gen_norm=None, loss_scale: float = 1.0,
              backward: bool = True, slot: str = "", first: bool = True, last: bool = True):
        from types import SimpleNamespace
        cfg = self.cfg
        S, L = b.S, cfg.num_layers
        self.loss_acc.zero_()
        if getattr(self, "_mode", None) is None or self._mode_S != S:
            self._mode, self._mode_S = self._pick_mode(S), S
            self._mode_steps = 0
        elif (self.recompute == "auto" and self._mode == "full" and self._mode_steps == 1 and backward
              and self.cp is None):       # context-parallel ranks must agree on the policy: no late change there
            # second step of an automatic "full" choice: every lazily allocated buffer now exists, so the free
            # memory is the steady-state figure; keep the attention outputs if they fit with room to spare
            free, _ = torch.cuda.mem_get_info(self.dev) if self.dev.type == "cuda" else (0, 0)
            per_attn = S * cfg.q_dim * 2 + cfg.num_heads * S * 4
            if free > L * per_attn + (12 << 30):
                self._mode = "attention"
        if backward:
            self._mode_steps = getattr(self, "_mode_steps", 0) + 1
        if self.cp is not None:
            if S != self.cp.S:
                raise ValueError(f"context-parallel attention was built for {self.cp.S} rows per rank, batch has {S}")
            self.cp.set_metadata(b.meta)
            plan = None
        else:
            plan = attn_ops.build_plan(b.meta)
        self._kb = b.group_range[:, 0].contiguous()
        self._ke = b.group_range[:, 1].contiguous()
        for gi in self.skip_wgrad_groups:
            # a frozen branch: its weight-gradient products get an empty row range and do no work
            self._ke[gi] = self._kb[gi]
        H = cfg.hidden_size
        st = SimpleNamespace(b=b, plan=plan, noise16=noise16, ce_norm=ce_norm, gen_norm=gen_norm, loss_scale=loss_scale,
                             backward=backward, slot=slot, first=first, last=last, kb=self._kb, ke=self._ke,
                             xs=[self.ws.get(f"{slot}x.{i}", (S, H)) for i in range(L + 1)],
                             saved_und=None, saved_gen=None, saved_t=None, saved_ns=None, z16=None, z_tok=None,
                             v_tok=None, d_last=None, d_first=None)
        return st

    def _fm_inputs(self, st):
        """Noised generation pixels ``z16`` of the micro-batch (deterministic in the batch's noise seed, so every
        pipeline stage that needs them derives the same values)."""
        if st.z16 is not None:
            return
        b, cfg = st.b, self.cfg
        m2 = cfg.merge_size ** 2
        if st.noise16 is None:
            gen = torch.Generator(device=self.dev).manual_seed(int(b.noise_seed))
            st.noise16 = torch.randn(b.gen_x16.shape, device=self.dev, generator=gen)
        t16 = b.gen_t.repeat_interleave(m2)[:, None]
        ns16 = b.gen_ns.repeat_interleave(m2)[:, None]
        st.z16 = t16 * b.gen_x16 + (1 - t16) * st.noise16 * ns16

    def embed_fwd(self, st):
        cfg, ws, p, b = self.cfg, self.ws, self.p, st.b
        x0 = st.xs[0]
        x0.zero_()
        self._need("front")
        if b.n_text:
            x0.index_copy_(0, b.text_rows, p["embed_tokens"].index_select(0, b.ids.index_select(0, b.text_rows).long()))
        sl = st.slot
        if b.und_rows.numel():
            emb, st.saved_und = self._vision_fwd("und", b.und_patches, b.und_px, b.und_py, sl + "vu")
            x0.index_copy_(0, b.und_rows, emb)
        if b.gen_rows.numel():
            self._fm_inputs(st)
            emb, st.saved_gen = self._vision_fwd("gen", st.z16.to(torch.bfloat16), b.gen_px, b.gen_py, sl + "vg")
            e_t, st.saved_t = self._scalar_embed_fwd("timestep_embedder", b.gen_t, sl + "te")
            emb = emb + e_t
            if cfg.add_noise_scale_embedding:
                e_n, st.saved_ns = self._scalar_embed_fwd("noise_scale_embedder", b.gen_ns / cfg.noise_scale_max_value,
                                                          sl + "ne")
                emb = emb + e_n
            x0.index_copy_(0, b.gen_rows, emb)

    def layers_fwd(self, st):
        self._kb, self._ke = st.kb, st.ke
        for l in range(self.cfg.num_layers):
            self._need(f"layer.{l}")
            self._layer_fwd(l, st.xs[l], st.xs[l + 1], st.b, st.plan)

    def heads(self, st):
        """Final norm, LM head + cross entropy, generation head + flow-matching loss (and the MTP heads); with
        ``st.backward`` also their gradients: ``st.d_last`` = d loss / d (last layer's output)."""
        cfg, ws, p, g, b = self.cfg, self.ws, self.p, self.g, st.b
        S, H, L = b.S, cfg.hidden_size, cfg.num_layers
        tg, xs, backward = b.tile_group, st.xs, st.backward
        ce_norm, gen_norm, loss_scale = st.ce_norm, st.gen_norm, st.loss_scale
        self._kb, self._ke = st.kb, st.ke
        self._need("head")
        if backward and self.on_backward_begin is not None:
            self.on_backward_begin()         # the heads below already write gradients
        Tg = b.gen_rows.numel()
        hf = ws.get("hf", (S, H)); rstd_f = ws.get("rstd_f", (S,), torch.float32)
        fused.rmsnorm_fwd(xs[L], p["final_norm"], tg, hf, rstd_f, cfg.rms_eps)
        d_hf = ws.get("d_hf", (S, H), zero=True)
        n_lab = b.label_rows.numel()
        if n_lab:
            norm = ce_norm if ce_norm is not None else max(b.ce_weight_sum, 1e-12)
            gscale = cfg.ce_loss_weight * loss_scale / norm
            h_sel = hf.index_select(0, b.label_rows)
            lab = b.labels.index_select(0, b.label_rows).contiguous()
            lw = b.loss_w.index_select(0, b.label_rows).contiguous()
            d_sel = ws.get("d_hsel", (n_lab, H))
            V = cfg.vocab_size
            for c0 in range(0, n_lab, self.ce_chunk):
                c1 = min(n_lab, c0 + self.ce_chunk)
                logits = gemm.gemm_nt(h_sel[c0:c1], p["lm_head"], out=ws.get("logits", (c1 - c0, V)))
                fused.ce_fwd_bwd(logits, lab[c0:c1], lw[c0:c1], gscale, self.loss_acc[0:4])
                if backward:
                    gemm.gemm_nn(logits, p["lm_head"], out=d_sel[c0:c1])
                    gemm.gemm_tn(logits, h_sel[c0:c1], out=g["lm_head"], out_mode=OUT_BF16_ACC)
            if backward:
                d_hf.index_copy_(0, b.label_rows, d_sel)
        if Tg:
            self._fm_inputs(st)
            x_tok = patches_to_tokens(b.gen_x16, cfg.patch_size, cfg.merge_size)
            z_tok = patches_to_tokens(st.z16, cfg.patch_size, cfg.merge_size).contiguous()
            v_tok = ((x_tok - z_tok) / (1 - b.gen_t[:, None]).clamp_min(cfg.t_eps)).contiguous()
            norm = gen_norm if gen_norm is not None else max(b.gen_weight_sum, 1.0)
            gscale = cfg.image_gen_loss_weight * loss_scale / norm
            h_gen = hf.index_select(0, b.gen_rows)
            ph = None
            if cfg.use_pixel_head:
                x_pred = ws.get("fm.xp", (Tg, cfg.token_dim))
                ph = self._pixel_head_fwd(h_gen.contiguous(), oracle.gen_image_grids(b), x_pred)
            else:
                a1 = self._linear(h_gen, p["fm_head.w1"], p["fm_head.b1"], out=ws.get("fm.a1", (Tg, cfg.fm_head_dim)))
                g1 = fused.gelu_fwd(a1, ws.get("fm.g1", (Tg, cfg.fm_head_dim)))
                x_pred = self._linear(g1, p["fm_head.w2"], p["fm_head.b2"], out=ws.get("fm.xp", (Tg, cfg.token_dim)))
            d_xp = ws.get("fm.dxp", (Tg, cfg.token_dim))
            row_loss = ws.get("fm.row_loss", (Tg,), torch.float32) if self.per_task_losses else None
            fused.fm_loss(x_pred, z_tok, v_tok, b.gen_t, b.gen_w, cfg.t_eps, gscale, d_xp, self.loss_acc[4:5],
                          row_loss=row_loss)
            if row_loss is not None:
                # weighted loss and weight per generation task (t2i 3, editing 4, interleave 5) for the log
                self.task_acc.zero_()
                tix = b.gen_task.long().clamp(0, 7)
                self.task_acc[0].index_add_(0, tix, row_loss * b.gen_w)
                self.task_acc[1].index_add_(0, tix, b.gen_w)
            if backward and ph is not None:
                d_hgen = ws.get("fm.dhgen", (Tg, H))
                self._pixel_head_bwd(d_xp, ph, d_hgen)
                d_hf.index_copy_(0, b.gen_rows, d_hgen)
            elif backward:
                self._wgrad(d_xp, g1, "fm_head.w2"); self._bgrad(d_xp, "fm_head.b2")
                d_g1 = gemm.gemm_nn(d_xp, p["fm_head.w2"], out=ws.get("fm.dg1", (Tg, cfg.fm_head_dim)))
                d_a1 = fused.gelu_bwd(a1, d_g1, d_g1)
                self._wgrad(d_a1, h_gen, "fm_head.w1"); self._bgrad(d_a1, "fm_head.b1")
                d_hgen = gemm.gemm_nn(d_a1, p["fm_head.w1"])
                d_hf.index_copy_(0, b.gen_rows, d_hgen)

        d_mtp = None
        if cfg.num_mtp_layers > 0:
            d_mtp = self._mtp(b, xs[L], st.plan, ce_norm, loss_scale, backward)
        out = self._losses(b, ce_norm, gen_norm)
        if not backward:
            return out
        self._ready("head")
        st.d_last = ws.get(st.slot + "dx.a", (S, H))
        fused.rmsnorm_bwd(d_hf, xs[L], p["final_norm"], rstd_f, tg, d_mtp, st.d_last, g["final_norm"])
        return out

    def layers_bwd(self, st):
        """Backward through this engine's decoder layers from ``st.d_last``; leaves ``st.d_first``."""
        ws, b = self.ws, st.b
        S, H, L = b.S, self.cfg.hidden_size, self.cfg.num_layers
        self._kb, self._ke = st.kb, st.ke
        cur = st.d_last
        bufs = [ws.get(st.slot + "dx.a", (S, H)), ws.get(st.slot + "dx.b", (S, H))]
        for l in range(L - 1, -1, -1):
            nxt = bufs[1] if cur.data_ptr() == bufs[0].data_ptr() else bufs[0]
            if self.on_layer_backward_begin is not None:
                self.on_layer_backward_begin(l)
            self._layer_bwd(l, st.xs[l], cur, nxt, b, st.plan)
            self._ready(f"layer.{l}")
            cur = nxt
        st.d_first = cur

    def embed_bwd(self, st):
        g, b = self.g, st.b
        dx0 = st.d_first
        if b.n_text:
            g["embed_tokens"].index_add_(0, b.ids.index_select(0, b.text_rows).long(), dx0.index_select(0, b.text_rows))
        if b.und_rows.numel():
            self._vision_bwd("und", dx0.index_select(0, b.und_rows), st.saved_und, st.slot + "vu")
        if b.gen_rows.numel():
            d_emb = dx0.index_select(0, b.gen_rows)
            self._vision_bwd("gen", d_emb, st.saved_gen, st.slot + "vg")
            self._scalar_embed_bwd("timestep_embedder", d_emb, st.saved_t)
            if st.saved_ns is not None:
                self._scalar_embed_bwd("noise_scale_embedder", d_emb, st.saved_ns)
        self._ready("front")

    def _mtp(self, b: PackedBatch, h_last, plan, ce_norm, loss_scale, backward):
        """Multi-token-prediction heads (reference training/sensenovalm/model/mtp.py:58-108): head k joins the
        hidden state of the previous depth with the embedding of the token k + 1 positions ahead
        (RMSNorm each, concatenate, project), runs one more decoder layer and predicts, through the shared final
        norm and LM head, the label k + 1 positions ahead of the main one; only text rows whose lookahead stays
        in the same run of text count.  Forward and backward of all heads; returns d loss / d ``h_last`` from
        the heads (None without backward).  The row selection is data dependent: one host read per head."""
        cfg, ws, p, g = self.cfg, self.ws, self.p, self.g
        if self.cp is not None:
            raise NotImplementedError("multi-token-prediction heads look ahead along the packed rows; with the "
                                      "rows of a sequence dealt over context-parallel ranks they are not supported")
        S, H = h_last.shape
        tg, V, eps = b.tile_group, cfg.vocab_size, cfg.rms_eps
        norm = ce_norm if ce_norm is not None else max(b.ce_weight_sum, 1e-12)
        gscale = cfg.mtp_loss_coeff * cfg.ce_loss_weight * loss_scale / norm
        idx = torch.arange(S, device=self.dev)
        doc, pos, text = b.meta[:, 0], b.meta[:, 1], b.kind == KIND_TEXT
        f32 = torch.float32
        st = []
        h = h_last
        for k in range(cfg.num_mtp_layers):
            tgt = (idx + k + 1).clamp_max(S - 1)
            ok = (idx + k + 1 < S) & text & text[tgt] & (doc[tgt] == doc) & (pos[tgt] == pos + k + 1)
            tok = b.ids.index_select(0, tgt).long()
            emb = (p["embed_tokens"].index_select(0, tok) * ok[:, None].to(torch.bfloat16)).contiguous()
            rs_h, rs_e = ws.get(f"mtp{k}.rsh", (S,), f32), ws.get(f"mtp{k}.rse", (S,), f32)
            nh = fused.rmsnorm_fwd(h, p[f"mtp.{k}.norm_hidden"], None, ws.get("mtp.nh", (S, H)), rs_h, eps)
            ne = fused.rmsnorm_fwd(emb, p[f"mtp.{k}.norm_embed"], None, ws.get("mtp.ne", (S, H)), rs_e, eps)
            z = ws.get(f"mtp{k}.z", (S, 2 * H))
            z[:, :H].copy_(nh)
            z[:, H:].copy_(ne)
            xin = gemm.gemm_nt(z, p[f"mtp.{k}.proj"], out=ws.get(f"mtp{k}.xin", (S, H)))
            hk = ws.get(f"mtp{k}.h", (S, H))
            self._layer_fwd(f"mtp.{k}.layer.", xin, hk, b, plan)
            rstd_f = ws.get(f"mtp{k}.rstdf", (S,), f32)
            hf = fused.rmsnorm_fwd(hk, p["final_norm"], tg, ws.get("mtp.hf", (S, H)), rstd_f, eps)
            lab_t, lw_t = b.labels.index_select(0, tgt), b.loss_w.index_select(0, tgt)
            rows = (ok & (lab_t >= 0) & (lw_t > 0)).nonzero().flatten()
            d_hf = ws.get(f"mtp{k}.dhf", (S, H), zero=True)
            n = int(rows.numel())
            if n:
                h_sel = hf.index_select(0, rows)
                lab = lab_t.index_select(0, rows).contiguous()
                lw = lw_t.index_select(0, rows).contiguous()
                d_sel = ws.get("mtp.dsel", (n, H))
                for c0 in range(0, n, self.ce_chunk):
                    c1 = min(n, c0 + self.ce_chunk)
                    logits = gemm.gemm_nt(h_sel[c0:c1], p["lm_head"], out=ws.get("logits", (c1 - c0, V)))
                    fused.ce_fwd_bwd(logits, lab[c0:c1], lw[c0:c1], gscale, self.loss_acc[8:12])
                    if backward:
                        gemm.gemm_nn(logits, p["lm_head"], out=d_sel[c0:c1])
                        gemm.gemm_tn(logits, h_sel[c0:c1], out=g["lm_head"], out_mode=OUT_BF16_ACC)
                if backward:
                    d_hf.index_copy_(0, rows, d_sel)
            st.append(dict(ok=ok, tok=tok, h_in=h, emb=emb, rs_h=rs_h, rs_e=rs_e, z=z, xin=xin, hk=hk,
                           rstd_f=rstd_f, d_hf=d_hf))
            h = hk
        if not backward:
            return None
        d_next = None                    # d loss / d h_k arriving from head k + 1
        for k in range(cfg.num_mtp_layers - 1, -1, -1):
            a = st[k]
            d_hk = fused.rmsnorm_bwd(a["d_hf"], a["hk"], p["final_norm"], a["rstd_f"], tg, d_next,
                                     ws.get("mtp.dhk", (S, H)), g["final_norm"])
            d_xin = ws.get("mtp.dxin", (S, H))
            self._layer_bwd(f"mtp.{k}.layer.", a["xin"], d_hk, d_xin, b, plan)
            dz = gemm.gemm_nn(d_xin, p[f"mtp.{k}.proj"], out=ws.get("mtp.dz", (S, 2 * H)))
            gemm.gemm_tn(d_xin, a["z"], out=g[f"mtp.{k}.proj"], out_mode=OUT_BF16_ACC)
            d_nh, d_ne = dz[:, :H].contiguous(), dz[:, H:].contiguous()
            d_prev = fused.rmsnorm_bwd(d_nh, a["h_in"], p[f"mtp.{k}.norm_hidden"], a["rs_h"], None, None,
                                       ws.get(f"mtp.dprev{k & 1}", (S, H)), g[f"mtp.{k}.norm_hidden"])
            d_emb = fused.rmsnorm_bwd(d_ne, a["emb"], p[f"mtp.{k}.norm_embed"], a["rs_e"], None, None,
                                      ws.get("mtp.demb", (S, H)), g[f"mtp.{k}.norm_embed"])
            okr = a["ok"].nonzero().flatten()
            if okr.numel():
                g["embed_tokens"].index_add_(0, a["tok"].index_select(0, okr), d_emb.index_select(0, okr))
            d_next = d_prev
        return d_next

    def _losses(self, b, ce_norm, gen_norm):
        cfg = self.cfg
        la = self.loss_acc
        ce_n = ce_norm if ce_norm is not None else max(b.ce_weight_sum, 1e-12)
        gn_n = gen_norm if gen_norm is not None else max(b.gen_weight_sum, 1.0)
        ce = la[0] / ce_n
        fm = la[4] / gn_n
        out = {"loss": cfg.ce_loss_weight * ce + cfg.image_gen_loss_weight * fm, "ce": ce, "fm": fm,
               "ce_correct": la[2].clone(), "ce_rows": la[3].clone()}      # copies: loss_acc is cleared per micro-batch
        if self.per_task_losses and b.gen_rows.numel():
            for tid, name in ((3, "t2i"), (4, "editing"), (5, "interleave")):
                out[f"image_gen_loss_{name}"] = self.task_acc[0, tid] / self.task_acc[1, tid].clamp_min(1e-12)
        if cfg.num_mtp_layers > 0:
            out["mtp"] = la[8] / ce_n
            out["loss"] = out["loss"] + cfg.mtp_loss_coeff * cfg.ce_loss_weight * out["mtp"]
        return out
