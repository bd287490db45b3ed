"""CUDA training engine of the MoE NEO-unify MoT model (A3B-MoT family): the dense engine
with the SwiGLU FFN of every layer replaced by two dropless top-k mixtures, one per branch
(understanding rows: ``num_experts``; generation rows: ``gen_num_experts``).

Routing never leaves the device (no split sizes on the host), tokens are laid out in expert
segments padded to the 128-row GEMM tile, and each projection of all experts of a branch is
one grouped tcgen05 GEMM launch.  Reference: QwenDroplessMoELayer
(training/sensenovalm/model/moe/dropless_layer_qwen.py:165-773), Qwen3MoeMoTDecoder MoE path
(training/sensenovalm/model/modeling_qwen3_moe_mot.py:372-393), load-balancing loss (:754-969).
"""
from __future__ import annotations

import torch

from ..data.batch import KIND_PAD, PackedBatch
from ..ops import fused, gemm, moe
from ..ops.gemm import OUT_BF16_ACC, OUT_F32_STORE
from .engine import MoTEngine


class MoEMoTEngine(MoTEngine):
    """``ep`` (a ``parallel.expert.ExpertParallel``): the experts are split over its ranks
    (``cfg.ep_size`` of them; the store then holds this rank's experts in the ``exp`` arena) and
    token rows are exchanged through peer memory."""

    def __init__(self, cfg, store, ep=None):
        if cfg.num_experts % 8 or cfg.gen_num_experts % 8:
            raise ValueError("expert counts must be multiples of 8 (gate GEMM tile granularity)")
        if (ep is None) != (cfg.ep_size <= 1) or (ep is not None and ep.world != cfg.ep_size):
            raise ValueError("cfg.ep_size and the expert-parallel group do not match")
        super().__init__(cfg, store)
        self.ep = ep
        self.aux_acc = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self.loss_scale_aux = 1.0
        self.monitor = None      # utils.moe_monitor.MoEMonitor: set to collect expert loads

    def _branches(self, b: PackedBatch):
        cfg = self.cfg
        # (name, row begin, row end, experts, top-k); under expert parallelism both mixtures always
        # take part (this rank's experts may receive rows even when it routes none itself)
        out = []
        if b.n_gen_pad > 0 or self.ep is not None:
            out.append(("gen", 0, b.n_gen_pad, cfg.gen_num_experts, cfg.gen_num_experts_per_tok))
        und_hi = self._und_hi
        if und_hi > b.n_gen_pad or self.ep is not None:
            out.append(("und", b.n_gen_pad, und_hi, cfg.num_experts, cfg.num_experts_per_tok))
        return out

    def forward_backward(self, b: PackedBatch, *a, **kw):
        self._und_hi = b.n_gen_pad + ((b.n_tokens - int(b.gen_rows.numel()) + 127) // 128) * 128
        self._row_valid = (b.kind != KIND_PAD).to(torch.int32)
        self._n_valid = {"gen": max(int(b.gen_rows.numel()), 1),
                         "und": max(b.n_tokens - int(b.gen_rows.numel()), 1)}
        self.aux_acc.zero_()
        out = super().forward_backward(b, *a, **kw)
        out["moe_aux"] = self.aux_acc[0].clone()
        out["loss"] = out["loss"] + self.cfg.router_aux_loss_coef * out["moe_aux"]
        return out

    def _ffn_fwd(self, l, h2, x1, out, b: PackedBatch, pn: str = ""):
        self._layer_idx = l
        if self.ep is not None:
            return self._ffn_fwd_ep(l, h2, x1, out, b)
        cfg, ws, p = self.cfg, self.ws, self.p
        s = self._pfx(l)
        H, Fe = cfg.hidden_size, cfg.moe_intermediate_size
        saved = {}
        for br, lo, hi, E, K in self._branches(b):
            R = hi - lo
            hb = h2[lo:hi]
            logits = gemm.gemm_nt(hb, p[s + f"moe_{br}.gate"], out=ws.get(f"moe.{br}.logits", (R, E), torch.float32),
                                  out_mode=OUT_F32_STORE)
            r = moe.route(logits, K, cfg.norm_topk_prob, self._row_valid[lo:hi].contiguous(),
                          bufs=_Prefixed(ws, f"moe.{br}."))
            xp = ws.get(f"moe.{br}.xp", (r.max_rows, H), zero=True)
            moe.gather(hb, r, xp)
            gu = gemm.gemm_nt(xp, p[s + f"moe_{br}.w13"], out=ws.get(f"moe.{br}.gu", (r.max_rows, 2 * Fe)),
                              tile_group=r.tile_group)
            act = fused.swiglu_fwd(gu, ws.get(f"moe.{br}.act", (r.max_rows, Fe)))
            yp = gemm.gemm_nt(act, p[s + f"moe_{br}.w2"], out=ws.get(f"moe.{br}.yp", (r.max_rows, H)),
                              tile_group=r.tile_group)
            if out is not None:
                moe.combine(yp, r, x1[lo:hi], out[lo:hi])
                if cfg.router_aux_loss_coef > 0:
                    self._aux_add(r, lo, hi, br, E, K)
            saved[br] = dict(r=r, xp=xp, gu=gu, act=act, yp=yp, lo=lo, hi=hi, E=E, K=K)
        if out is not None and self._und_hi < out.shape[0]:
            out[self._und_hi:].copy_(x1[self._und_hi:])          # padding-only tiles
        return dict(moe=saved)

    def _aux_add(self, r, lo, hi, br, E, K):
        if self.monitor is not None:
            self.monitor.record(self._layer_idx, br, r.counts)
        nv = self._n_valid[br]
        valid = self._row_valid[lo:hi].bool()
        Pm = (r.probs * valid[:, None]).sum(0) / nv
        f = r.counts.float() / (nv * K)
        self.aux_acc += E * (f * Pm).sum()

    # ---- expert parallel: phases separated by device-side flag barriers ------------------------
    def _ffn_fwd_ep(self, l, h2, x1, out, b: PackedBatch):
        cfg, ws, p, ep = self.cfg, self.ws, self.p, self.ep
        s = self._pfx(l)
        H, Fe = cfg.hidden_size, cfg.moe_intermediate_size
        saved = {}
        # phase 1: route locally, clear my receive buffers, publish my per-expert counts to every rank
        for br, lo, hi, E, K in self._branches(b):
            R = hi - lo
            eb = ep.bufs[br]
            r = None
            if R > 0:
                hb = h2[lo:hi]
                logits = gemm.gemm_nt(hb, p[s + f"moe_{br}.gate"], out=ws.get(f"moe.{br}.logits", (R, E), torch.float32),
                                      out_mode=OUT_F32_STORE)
                r = moe.route(logits, K, cfg.norm_topk_prob, self._row_valid[lo:hi].contiguous(),
                              bufs=_Prefixed(ws, f"moe.{br}."), layout=False)
                counts = r.counts
            else:
                counts = ws.get(f"moe.{br}.zero_counts", (E,), torch.int32, zero=True)
            moe.ep_put_counts(counts, eb.counts_all.c_ptrs, ep.world, ep.rank, E)
            saved[br] = dict(r=r, lo=lo, hi=hi, E=E, K=K, R=R)
        ep.barrier()
        # phase 2: everyone derives the same layout; rows go to the owners' buffers by peer stores
        for br, sv in saved.items():
            eb, r = ep.bufs[br], sv["r"]
            er = moe.ep_plan(eb.counts_all.tensor, ep.world, ep.rank, sv["E"], eb.capacity,
                             r.top_idx if r is not None else None, r.top_w if r is not None else None,
                             sv["R"], sv["K"], _Prefixed(ws, f"moe.{br}."))
            # padding rows of my receive buffers (nobody writes them; the weight-gradient GEMMs read them)
            moe.ep_zero_pads(er, eb.view("xp"), eb.view("dyp"))
            moe.ep_dispatch(h2[sv["lo"]:sv["hi"]], er, eb.xp.c_ptrs)
            sv["er"] = er
        ep.barrier()
        # phase 3: my experts on everything that arrived (grouped GEMMs over the local segments)
        for br, sv in saved.items():
            eb, er = ep.bufs[br], sv["er"]
            xp = eb.view("xp")
            gu = gemm.gemm_nt(xp, p[s + f"moe_{br}.w13"], out=ws.get(f"moe.{br}.gu", (eb.capacity, 2 * Fe)),
                              tile_group=er.tile_group, rows_dev=er.total_rows)
            act = fused.swiglu_fwd(gu, ws.get(f"moe.{br}.act", (eb.capacity, Fe)), rows_dev=er.total_rows)
            gemm.gemm_nt(act, p[s + f"moe_{br}.w2"], out=eb.view("yp"), tile_group=er.tile_group,
                         rows_dev=er.total_rows)
            sv.update(xp=xp, gu=gu, act=act)
        if out is not None:
            ep.barrier()
            # phase 4: pull my rows' expert outputs back from the owners
            for br, sv in saved.items():
                lo, hi = sv["lo"], sv["hi"]
                if sv["R"] == 0:
                    continue
                moe.ep_combine(ep.bufs[br].yp.c_ptrs, sv["er"], sv["r"].top_w, x1[lo:hi], out[lo:hi])
                if cfg.router_aux_loss_coef > 0:
                    self._aux_add(sv["r"], lo, hi, br, sv["E"], sv["K"])
            if self._und_hi < out.shape[0]:
                out[self._und_hi:].copy_(x1[self._und_hi:])
        return dict(moe=saved)

    def _ffn_bwd_ep(self, l, a, dy, b: PackedBatch):
        cfg, ws, p, g, ep = self.cfg, self.ws, self.p, self.g, self.ep
        s = self._pfx(l)
        S, H = dy.shape
        Fe = cfg.moe_intermediate_size
        d_h2 = ws.get("d_h", (S, H), zero=True)
        ep.barrier()          # every owner's yp is complete and its dyp is cleared
        for br, sv in a["moe"].items():
            if sv["R"] == 0:
                continue
            eb = ep.bufs[br]
            sv["dw"] = ws.get(f"moe.{br}.dw", (sv["R"], sv["K"]), torch.float32)
            moe.ep_combine_bwd(dy[sv["lo"]:sv["hi"]], eb.yp.c_ptrs, eb.dyp.c_ptrs, sv["er"], sv["dw"])
        ep.barrier()
        for br, sv in a["moe"].items():
            eb, er = ep.bufs[br], sv["er"]
            d_yp = eb.view("dyp")
            d_act = gemm.gemm_nn(d_yp, p[s + f"moe_{br}.w2"], out=ws.get(f"moe.{br}.d_act", (eb.capacity, Fe)),
                                 tile_group=er.tile_group, rows_dev=er.total_rows)
            gemm.gemm_tn(d_yp, sv["act"], out=g[s + f"moe_{br}.w2"], k_begin=er.seg_start, k_end=er.seg_end,
                         num_groups=er.E_loc, out_mode=OUT_BF16_ACC)
            d_gu = fused.swiglu_bwd(sv["gu"], d_act, ws.get(f"moe.{br}.d_gu", (eb.capacity, 2 * Fe)),
                                    rows_dev=er.total_rows)
            gemm.gemm_nn(d_gu, p[s + f"moe_{br}.w13"], out=eb.view("dxp"), tile_group=er.tile_group,
                         rows_dev=er.total_rows)
            gemm.gemm_tn(d_gu, sv["xp"], out=g[s + f"moe_{br}.w13"], k_begin=er.seg_start, k_end=er.seg_end,
                         num_groups=er.E_loc, out_mode=OUT_BF16_ACC)
        ep.barrier()
        for br, sv in a["moe"].items():
            if sv["R"] == 0:
                continue
            r, lo, hi, E, K, R = sv["r"], sv["lo"], sv["hi"], sv["E"], sv["K"], sv["R"]
            moe.ep_combine(ep.bufs[br].dxp.c_ptrs, sv["er"], None, None, d_h2[lo:hi])
            nv = self._n_valid[br]
            aux_scale = cfg.router_aux_loss_coef * self._aux_grad_scale * E / (float(nv) * K * nv)
            dlog = moe.router_bwd(r, sv["dw"], aux_scale, cfg.norm_topk_prob, ws.get(f"moe.{br}.dlog", (R, E)))
            gemm.gemm_nn(dlog, p[s + f"moe_{br}.gate"], out=d_h2[lo:hi], out_mode=OUT_BF16_ACC)
            gemm.gemm_tn(dlog, a["h2"][lo:hi], out=g[s + f"moe_{br}.gate"], out_mode=OUT_BF16_ACC)
        return d_h2

    def _ffn_bwd(self, l, a, dy, b: PackedBatch):
        if self.ep is not None:
            return self._ffn_bwd_ep(l, a, dy, b)
        cfg, ws, p, g = self.cfg, self.ws, self.p, self.g
        s = self._pfx(l)
        S, H = dy.shape
        Fe = cfg.moe_intermediate_size
        d_h2 = ws.get("d_h", (S, H), zero=True)
        for br, sv in a["moe"].items():
            r, lo, hi, E, K = sv["r"], sv["lo"], sv["hi"], sv["E"], sv["K"]
            R = hi - lo
            d_yp = ws.get(f"moe.{br}.d_yp", (r.max_rows, H), zero=True)
            dw = ws.get(f"moe.{br}.dw", (R, K), torch.float32)
            moe.combine_bwd(dy[lo:hi], sv["yp"], r, d_yp, dw)
            d_act = gemm.gemm_nn(d_yp, p[s + f"moe_{br}.w2"], out=ws.get(f"moe.{br}.d_act", (r.max_rows, Fe)),
                                 tile_group=r.tile_group)
            gemm.gemm_tn(d_yp, sv["act"], out=g[s + f"moe_{br}.w2"], k_begin=r.seg_start, k_end=r.seg_end,
                         num_groups=E, out_mode=OUT_BF16_ACC)
            d_gu = fused.swiglu_bwd(sv["gu"], d_act, ws.get(f"moe.{br}.d_gu", (r.max_rows, 2 * Fe)))
            d_xp = gemm.gemm_nn(d_gu, p[s + f"moe_{br}.w13"], out=ws.get(f"moe.{br}.d_xp", (r.max_rows, H)),
                                tile_group=r.tile_group)
            gemm.gemm_tn(d_gu, sv["xp"], out=g[s + f"moe_{br}.w13"], k_begin=r.seg_start, k_end=r.seg_end,
                         num_groups=E, out_mode=OUT_BF16_ACC)
            moe.gather_bwd(d_xp, r, d_h2[lo:hi])
            nv = self._n_valid[br]
            aux_scale = cfg.router_aux_loss_coef * self._aux_grad_scale * E / (float(nv) * K * nv)
            dlog = moe.router_bwd(r, dw, aux_scale, cfg.norm_topk_prob, ws.get(f"moe.{br}.dlog", (R, E)))
            hb = a["h2"][lo:hi]
            gemm.gemm_nn(dlog, p[s + f"moe_{br}.gate"], out=d_h2[lo:hi], out_mode=OUT_BF16_ACC)
            gemm.gemm_tn(dlog, hb, out=g[s + f"moe_{br}.gate"], out_mode=OUT_BF16_ACC)
        return d_h2

    _aux_grad_scale = 1.0


class _Prefixed:
    """Workspace view that prefixes buffer names (one set of routing buffers per branch)."""

    def __init__(self, ws, prefix):
        self.ws, self.prefix = ws, prefix

    def get(self, name, shape, dtype, **kw):
        return self.ws.get(self.prefix + name, shape, dtype, **kw)
