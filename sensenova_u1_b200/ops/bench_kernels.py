"""Single-kernel timings (CUDA events, L2 flushed between iterations) for the hot ops, and the
small cases that profiler captures are taken on:

    python -m sensenova_u1_b200.ops.bench_kernels --kernel gemm_w13 --iters 5
    python -m sensenova_u1_b200.ops.bench_kernels --kernel attn_fwd --iters 3

Kernels: gemm_w13 / gemm_w2 / gemm_qkv (8B-MoT projection shapes at 16384 rows, grouped by MoT
branch), gemm_wgrad (dy^T x), attn_fwd / attn_bwd (causal packed documents, 32 query / 8 kv heads,
head 128), rmsnorm, qknorm_rope, swiglu, adamw.  Prints one JSON line per kernel with the time,
achieved TFLOP/s or GB/s and the fraction of the measured peaks when MEASURED_PEAKS.json is present.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d.get("bf16_tflops", 1590.0)), float(d.get("hbm_gbs", 6650.0)), "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.add_(1.0)                      # > L2: evicts the operands of the previous iteration
        a, b = torch.cuda.Event(True), torch.cuda.Event(True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--adamw-n", type=int, default=1 << 28, help="elements of the AdamW timing")
    ap.add_argument("--adamw-state", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--single-cta", action="store_true",
                    help="GEMMs on the single-CTA kernel (128x256 tiles) instead of the two-SM pair kernel")
    ap.add_argument("--pair-band", type=int, default=0, help="pair tiles per scheduling band (0: library default)")
    args = ap.parse_args()
    from . import attention, fused, gemm
    from ._lib import check_status
    dev = torch.device("cuda")
    torch.manual_seed(0)
    S, H, F, QKV = args.rows, 4096, 12288, 6144
    flush = torch.zeros(256 << 20, dtype=torch.float32, device=dev)      # 1 GiB
    tf_peak, bw_peak, src = _peaks()
    tg = torch.zeros(S // 128, dtype=torch.int32, device=dev)
    tg[S // 256:] = 1
    rnd = lambda *s: (torch.randn(*s, device=dev) * 0.05).to(torch.bfloat16)
    out = []

    def report(name, ms, flops=None, nbytes=None):
        r = {"kernel": name, "ms": round(ms, 4)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r[f"of_{src}_bf16_peak"] = round(flops / ms / 1e9 / tf_peak, 3)
        if nbytes:
            r["gbs"] = round(nbytes / ms / 1e6, 1)
            r[f"of_{src}_hbm_copy"] = round(nbytes / ms / 1e6 / bw_peak, 3)
        print(json.dumps(r), flush=True)
        out.append(r)

    want = lambda k: args.kernel in ("all", k)
    if args.single_cta:
        gemm.set_pair_mode(False)
    if args.pair_band:
        from . import _lib as _l
        _l.load().snu1_gemm_set_pair_band(args.pair_band)
    x = rnd(S, H)
    for name, n, k in (("gemm_w13", 2 * F, H), ("gemm_qkv", QKV, H), ("gemm_w2", H, F)):
        if not want(name):
            continue
        xin = x if k == H else rnd(S, k)
        w = rnd(2, n, k)
        y = torch.empty(S, n, dtype=torch.bfloat16, device=dev)
        ms = _time(lambda: gemm.gemm_nt(xin, w, out=y, tile_group=tg), args.iters, flush)
        report(name, ms, flops=2.0 * S * n * k)
    if want("gemm_dgrad"):
        dy = rnd(S, 2 * F)
        w = rnd(2, 2 * F, H)
        dx = torch.empty(S, H, dtype=torch.bfloat16, device=dev)
        ms = _time(lambda: gemm.gemm_nn(dy, w, out=dx, tile_group=tg), args.iters, flush)
        report("gemm_dgrad", ms, flops=2.0 * S * 2 * F * H)
    if want("gemm_wgrad"):
        dy = rnd(S, 2 * F)
        gw = torch.zeros(2, 2 * F, H, dtype=torch.bfloat16, device=dev)
        kb = torch.tensor([0, S // 2], dtype=torch.int32, device=dev)
        ke = torch.tensor([S // 2, S], dtype=torch.int32, device=dev)
        ms = _time(lambda: gemm.gemm_tn(dy, x, out=gw, k_begin=kb, k_end=ke, num_groups=2,
                                        out_mode=gemm.OUT_BF16_ACC), args.iters, flush)
        report("gemm_wgrad", ms, flops=2.0 * S * 2 * F * H)
    if want("attn_fwd") or want("attn_bwd"):
        Hq, Hk, D = 32, 8, 128
        q, k, v = rnd(S, Hq, D) * 10, rnd(S, Hk, D) * 10, rnd(S, Hk, D) * 10
        meta = attention.make_meta(torch.zeros(S, dtype=torch.int32), torch.arange(S, dtype=torch.int32)).to(dev)
        plan = attention.build_plan(meta, meta)
        o = torch.empty_like(q)
        lse = torch.empty(Hq, S, dtype=torch.float32, device=dev)
        scale = D ** -0.5
        flops = 4.0 * Hq * S * S * D / 2          # causal
        if want("attn_fwd"):
            ms = _time(lambda: attention.attention_fwd(q, k, v, plan, scale, out=o, lse=lse), args.iters, flush)
            report("attn_fwd", ms, flops=flops)
        if want("attn_bwd"):
            attention.attention_fwd(q, k, v, plan, scale, out=o, lse=lse)
            do = rnd(S, Hq, D)
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            ms = _time(lambda: attention.attention_bwd(q, k, v, o, do, lse, plan, scale, dq=dq, dk=dk, dv=dv),
                       args.iters, flush)
            report("attn_bwd", ms, flops=2.5 * flops)
    if args.kernel in ("attn_packed",):
        # The training step's real mix: a packed multimodal batch (documents of 1-4 k tokens with images, rows in
        # [generation | understanding] order), 32 / 8 heads.  FLOPs are counted over the (query, key) pairs the mask
        # allows; "tile_tflops" counts whole kept tiles (what the kernels actually multiply).
        from ..config import get_config
        from ..data.synthetic import synthetic_batch
        Hq, Hk, D = 32, 8, 128
        b = synthetic_batch(get_config("8b-mot"), S, seed=0).to(dev)
        plan = attention.build_plan(b.meta)
        kept = int((plan.cls != 0).sum())
        partial = int((plan.cls == 1).sum())
        pairs = 0
        for r0 in range(0, S, 4096):                      # dense mask in row slabs
            pairs += int(attention.dense_mask(b.meta[r0:r0 + 4096], b.meta).sum())
        q, k, v = rnd(S, Hq, D) * 10, rnd(S, Hk, D) * 10, rnd(S, Hk, D) * 10
        o = torch.empty_like(q)
        lse = torch.empty(Hq, S, dtype=torch.float32, device=dev)
        scale = D ** -0.5
        flops, tile_flops = 4.0 * Hq * pairs * D, 4.0 * Hq * kept * 128 * 128 * D
        ms_f = _time(lambda: attention.attention_fwd(q, k, v, plan, scale, out=o, lse=lse), args.iters, flush)
        do = rnd(S, Hq, D)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ms_b = _time(lambda: attention.attention_bwd(q, k, v, o, do, lse, plan, scale, dq=dq, dk=dk, dv=dv),
                     args.iters, flush)
        for name, ms, mult in (("attn_packed_fwd", ms_f, 1.0), ("attn_packed_bwd", ms_b, 2.5)):
            print(json.dumps({"kernel": name, "rows": S, "kept_tiles": kept, "partial_tiles": partial,
                              "mask_density": round(pairs / float(S) / S, 4), "ms": round(ms, 3),
                              "tflops": round(mult * flops / ms / 1e9, 1),
                              "tile_tflops": round(mult * tile_flops / ms / 1e9, 1)}), flush=True)
    if args.kernel in ("prefill_hybrid",):
        # Hybrid-mask prefill (causal text + bidirectional image spans), the shapes of the reference's
        # published kernel table (docs/inference_infra.md:52-68: batch, max_seq_len, image_token_num ->
        # Triton ms / FA3 ms on H100).  The table does not give the actual lengths; every sequence is
        # taken at max_seq_len here, an upper bound on the work of the published row.
        Hq, Hk, D = 32, 8, 128
        published = {(8, 4096, 88): (1.95, 0.81), (8, 8192, 171): (6.55, 2.68), (16, 4096, 379): (4.12, 1.68),
                     (16, 8192, 246): (17.76, 7.40), (32, 4096, 726): (8.46, 3.46)}
        for (B, L, n_img), (t_triton, t_fa3) in published.items():
            Sx = B * L
            doc = torch.arange(Sx, dtype=torch.int32) // L
            pos = torch.arange(Sx, dtype=torch.int32) % L
            span = max(1, n_img // B)
            in_img = (pos >= 16) & (pos < 16 + span)              # one bidirectional image span per sequence
            img = torch.where(in_img, doc + 1, torch.zeros_like(doc))
            pos_m = torch.where(in_img, torch.full_like(pos, 16), torch.where(pos >= 16 + span, pos - span + 1, pos))
            meta = attention.make_meta(doc, pos_m, img).to(dev)
            plan = attention.build_plan(meta, meta)
            q, k, v = rnd(Sx, Hq, D) * 10, rnd(Sx, Hk, D) * 10, rnd(Sx, Hk, D) * 10
            o = torch.empty_like(q)
            lse = torch.empty(Hq, Sx, dtype=torch.float32, device=dev)
            ms = _time(lambda: attention.attention_fwd(q, k, v, plan, D ** -0.5, out=o, lse=lse), args.iters, flush)
            r = {"kernel": "prefill_hybrid", "batch": B, "seq_len": L, "image_tokens": n_img, "ms": round(ms, 3),
                 "tflops": round(4.0 * Hq * B * L * L * D / 2 / ms / 1e9, 1),
                 "published_h100_ms_unknown_lengths": {"triton": t_triton, "fa3": t_fa3}}
            print(json.dumps(r), flush=True)
            del q, k, v, o, lse
    if want("rmsnorm"):
        gain = torch.ones(2, H, device=dev)
        y = torch.empty_like(x)
        rstd = torch.empty(S, dtype=torch.float32, device=dev)
        ms = _time(lambda: fused.rmsnorm_fwd(x, gain, tg, y, rstd, 1e-6), args.iters, flush)
        report("rmsnorm_fwd", ms, nbytes=2.0 * S * H * 2)
    if want("swiglu"):
        gu = rnd(S, 2 * F)
        act = torch.empty(S, F, dtype=torch.bfloat16, device=dev)
        ms = _time(lambda: fused.swiglu_fwd(gu, act), args.iters, flush)
        report("swiglu_fwd", ms, nbytes=3.0 * S * F * 2)
    if want("adamw"):
        n = args.adamw_n
        sdt = torch.float32 if args.adamw_state == "fp32" else torch.bfloat16
        p = torch.zeros(n, dtype=torch.bfloat16, device=dev)
        lo = torch.zeros(n, dtype=torch.int16, device=dev)
        g = torch.zeros(n, dtype=torch.bfloat16, device=dev)
        m = torch.zeros(n, dtype=sdt, device=dev)
        v = torch.zeros(n, dtype=sdt, device=dev)
        nsq = torch.ones(1, dtype=torch.float32, device=dev)
        sk = torch.zeros(1, dtype=torch.int32, device=dev)
        ms = _time(lambda: fused.adamw(p, lo, g, m, v, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0,
                                       step=1, grad_prescale=1.0, norm_sq=nsq, max_norm=1.0, skipped=sk),
                   args.iters, flush)
        sb = 4 if args.adamw_state == "fp32" else 2
        report(f"adamw_{args.adamw_state}_moments_{n >> 20}Mi", ms, nbytes=n * (6.0 + 2 * sb) + n * (4.0 + 2 * sb))
    check_status()


if __name__ == "__main__":
    main()
