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

from ..data.batch import KIND_PAD, KIND_UND_IMG, PackedBatch
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
        self.z_acc = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self.loss_scale_aux = 1.0
        # bias-based balancing (reference: e_score_correction_bias, model/moe/dropless_layer_qwen.py:90-163, updated
        # once per step from the accumulated expert counts, core/scheduler/no_pipeline_scheduler.py:320-332,
        # utils/common.py:501-517): one selection bias per (layer, branch, expert), not trained by the optimizer;
        # :meth:`update_selection_bias` moves each by +-router_bias_update_rate towards the mean load
        self.sel_bias, self.sel_counts = {}, {}
        if cfg.router_bias_update_rate > 0:
            for l in range(cfg.num_layers):
                for br, E in (("gen", cfg.gen_num_experts), ("und", cfg.num_experts)):
                    self.sel_bias[(l, br)] = torch.zeros(E, dtype=torch.float32, device=self.dev)
                    self.sel_counts[(l, br)] = torch.zeros(E, dtype=torch.float32, device=self.dev)
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
        cfg = self.cfg
        self._class_split = cfg.moe_balance_image_ratio > 0 or cfg.moe_balance_text_ratio > 0
        self._row_class = (b.kind == KIND_UND_IMG).to(torch.int32) if self._class_split else None
        if self._class_split:
            n_img = int((b.kind == KIND_UND_IMG).sum())
            n_und = b.n_tokens - int(b.gen_rows.numel())
            self._n_class = (max(n_und - n_img, 1), max(n_img, 1))          # (text, image) rows of the und branch
        self.z_acc.zero_()
        self._n_valid = {"gen": max(int(b.gen_rows.numel()), 1),
                         "und": max(b.n_tokens - int(b.gen_rows.numel()), 1)}
        self.aux_acc.zero_()
        out = super().forward_backward(b, *a, **kw)
        out["moe_aux"] = self.aux_acc[0].clone()
        out["loss"] = out["loss"] + self.cfg.router_aux_loss_coef * out["moe_aux"]
        if self.cfg.router_z_loss_coef > 0:
            out["moe_z_loss"] = self.z_acc[0].clone()
            out["loss"] = out["loss"] + self.cfg.router_z_loss_coef * out["moe_z_loss"]
        return out

    def _route(self, logits, K, lo, hi, br, bufs, layout=True):
        """Routing of one branch's rows with the configured training extras."""
        cfg = self.cfg
        l = self._layer_idx
        bias = self.sel_bias.get((l, br)) if isinstance(l, int) else None
        rc = self._row_class[lo:hi].contiguous() if (self._class_split and br == "und") else None
        return moe.route(logits, K, cfg.norm_topk_prob, self._row_valid[lo:hi].contiguous(), bufs=bufs, layout=layout,
                         sel_bias=bias, want_lse=cfg.router_z_loss_coef > 0, row_class=rc)

    def _router_bwd(self, r, dw, br, E, K, dlogits):
        cfg = self.cfg
        nv = self._n_valid[br]
        base = cfg.router_aux_loss_coef * self._aux_grad_scale * E * self._branch_ratio(br)
        aux_scale = base / (float(nv) * K * nv)
        scales = None
        if r.class_counts is not None:
            nt, ni = self._n_class
            scales = (cfg.moe_balance_text_ratio * base / (float(nt) * K * nt),
                      cfg.moe_balance_image_ratio * base / (float(ni) * K * ni))
        z = cfg.router_z_loss_coef * self._aux_grad_scale / float(nv) if r.lse is not None else 0.0
        return moe.router_bwd(r, dw, aux_scale, cfg.norm_topk_prob, dlogits, class_scales=scales, z_scale=z)

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
            r = self._route(logits, K, lo, hi, br, _Prefixed(ws, f"moe.{br}."))
            xp = ws.get(f"moe.{br}.xp", (r.max_rows, H), zero=True)
            moe.gather(hb, r, xp)
            gu = gemm.gemm_nt(xp, p[s + f"moe_{br}.w13"], out=ws.get(f"moe.{br}.gu", (r.max_rows, 2 * Fe)),
                              tile_group=r.tile_group)
            act = fused.swiglu_fwd(gu, ws.get(f"moe.{br}.act", (r.max_rows, Fe)))
            yp = gemm.gemm_nt(act, p[s + f"moe_{br}.w2"], out=ws.get(f"moe.{br}.yp", (r.max_rows, H)),
                              tile_group=r.tile_group)
            if out is not None:
                moe.combine(yp, r, x1[lo:hi], out[lo:hi])
                self._count_selected(r, br)
                if cfg.router_aux_loss_coef > 0:
                    self._aux_add(r, lo, hi, br, E, K)
            saved[br] = dict(r=r, xp=xp, gu=gu, act=act, yp=yp, lo=lo, hi=hi, E=E, K=K)
        if out is not None and self._und_hi < out.shape[0]:
            out[self._und_hi:].copy_(x1[self._und_hi:])          # padding-only tiles
        return dict(moe=saved)

    def _count_selected(self, r, br):
        """Forward pass only (not the recomputation in backward): expert loads for the bias update of the step."""
        cnt = self.sel_counts.get((self._layer_idx, br)) if isinstance(self._layer_idx, int) else None
        if cnt is not None:
            cnt.add_(r.counts.float())

    def _branch_ratio(self, br: str) -> float:
        """Weight of a mixture's balance loss in the sum (``moe_balance_gen_ratio`` / ``moe_balance_und_ratio``)."""
        return float(self.cfg.moe_balance_gen_ratio if br == "gen" else self.cfg.moe_balance_und_ratio)

    def _aux_add(self, r, lo, hi, br, E, K):
        if self.monitor is not None:
            self.monitor.record(self._layer_idx, br, r.counts)
        nv = self._n_valid[br]
        valid = self._row_valid[lo:hi].bool()
        cfg = self.cfg
        if r.class_counts is not None:
            # text and image tokens of the understanding branch balanced separately, mixed with the configured ratios
            # (reference: load_balancing_loss_func with image_inds, modeling_qwen3_moe_mot.py:824-920)
            for c, ratio, n in ((0, cfg.moe_balance_text_ratio, self._n_class[0]),
                                (1, cfg.moe_balance_image_ratio, self._n_class[1])):
                m = valid & (r.row_class == c)
                Pm = (r.probs * m[:, None]).sum(0) / n
                f = r.class_counts[c].float() / (n * K)
                self.aux_acc += self._branch_ratio(br) * ratio * E * (f * Pm).sum()
        else:
            Pm = (r.probs * valid[:, None]).sum(0) / nv
            f = r.counts.float() / (nv * K)
            self.aux_acc += self._branch_ratio(br) * E * (f * Pm).sum()
        if r.lse is not None:
            self.z_acc += (r.lse * valid).pow(2).sum() / nv

    def update_selection_bias(self, group=None) -> None:
        """End of a step: every selection bias moves one signed step of ``router_bias_update_rate`` towards the mean
        load of its mixture, from the counts accumulated over the step's micro-batches (summed over ``group`` first
        when given, so that data-parallel ranks keep identical biases), then the counts are cleared."""
        if not self.sel_bias:
            return
        keys = sorted(self.sel_bias)
        flat = torch.cat([self.sel_counts[k] for k in keys])
        if group is not None and torch.distributed.is_initialized() and torch.distributed.get_world_size(group) > 1:
            torch.distributed.all_reduce(flat, group=group)
        off = 0
        rate = self.cfg.router_bias_update_rate
        for k in keys:
            n = self.sel_counts[k].numel()
            load = flat[off:off + n]
            self.sel_bias[k].add_(rate * torch.sign(load.mean() - load))
            self.sel_counts[k].zero_()
            off += n

    def selection_bias_state(self) -> dict:
        return {f"{l}.{br}": t.detach().cpu() for (l, br), t in self.sel_bias.items()}

    def load_selection_bias_state(self, sd: dict) -> None:
        for (l, br), t in self.sel_bias.items():
            v = sd.get(f"{l}.{br}")
            if v is not None:
                t.copy_(v.to(t.device, t.dtype))

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
                r = self._route(logits, K, lo, hi, br, _Prefixed(ws, f"moe.{br}."), layout=False)
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
                self._count_selected(sv["r"], br)
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
            dlog = self._router_bwd(r, sv["dw"], br, E, K, ws.get(f"moe.{br}.dlog", (R, E)))
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
            dlog = self._router_bwd(r, dw, br, E, K, ws.get(f"moe.{br}.dlog", (R, E)))
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
