"""CUDA inference engine of the NEO-unify MoT model: prefix (understanding branch)
forward with KV cache, flow-matching image denoising through the generation branch,
and greedy text decoding — all on the sm_100a kernels of this package.

Differences from the reference's generation loops
(src/sensenova_u1/models/neo_unify/modeling_neo_chat.py:1691-1860, modeling_qwen3.py:583-745):
the conditional and unconditional branches run as two documents of ONE packed forward
(one GEMM launch per projection instead of two passes), the prefix attention uses the
tile-classified tensor-core kernel instead of eager fp32 softmax, K/V of the prefix stay
in place in a per-layer buffer and only the image rows are rewritten each step, and the
CFG combine + Euler step + re-patchify are one kernel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..config import ModelConfig
from ..data.batch import apply_time_schedule
from ..models import oracle
from ..models.engine import Workspace
from ..models.params import GEN, UND, ParamStore
from ..ops import _lib, attention as attn_ops, fused, gemm
from ..ops._lib import c_float, c_int, c_void_p

CFG_NORMS = {"none": 0, "global": 1, "channel": 2, "cfg_zero_star": 3}


def _pad128(n):
    return (n + 127) // 128 * 128


@dataclass
class DocLayout:
    """Row ranges of one document inside the per-layer KV buffer."""
    kv_start: int      # first KV row of the document
    prefix_len: int    # text / understanding rows already cached
    img_start: int     # first row reserved for the image being generated
    next_pos: int      # t index the next token / image takes


class InferenceEngine:
    def __init__(self, cfg: ModelConfig, store: ParamStore, offload=None):
        """``offload``: a ``utils.offload.LayerOffloader``; the decoder-layer weights then come from it
        (streamed from pinned host memory one layer ahead) and ``store`` only needs the other tensors."""
        if cfg.head_dim != 128:
            raise ValueError("the sm_100a attention kernels need head_dim 128")
        self.cfg, self.store, self.p = cfg, store, store.p
        self.offload = offload
        self.dev = store.device
        self.ws = Workspace(self.dev)
        inv_t, inv_hw = oracle.rope_inv_freq(cfg, self.dev)
        self.inv_t, self.inv_hw = inv_t.contiguous(), inv_hw.contiguous()
        half = cfg.vision_hidden // 2
        self.inv_v = (1.0 / (cfg.rope_theta_vision ** (
            torch.arange(0, half, 2, dtype=torch.float32, device=self.dev) / half))).contiguous()
        self.scale = cfg.head_dim ** -0.5
        self.kc: List[torch.Tensor] = []
        self.vc: List[torch.Tensor] = []
        self.stats = torch.zeros(4 + 4 * 592, dtype=torch.float32, device=self.dev)   # sums + per-block partials
        self.sp = None      # sequence-parallel sampling state (enable_sequence_parallel)

    def enable_sequence_parallel(self, group) -> None:
        """Splits the image tokens of :meth:`denoise` over the ranks of ``group`` (all of which run the same
        call with the same arguments).  The per-layer K/V caches move to symmetric memory: every rank writes
        the keys / values of its token slice into all peers' caches with peer stores, a device-side flag
        barrier per layer orders the writes before the attention reads.  Call before the first prefill."""
        import torch.distributed as dist
        from ..parallel.symm import FlagBarrier
        self.sp = {"group": group, "world": dist.get_world_size(group), "rank": dist.get_rank(group),
                   "bar": FlagBarrier(group, self.dev), "k": None, "v": None}
        self.kc, self.vc = [], []

    # ------------------------------------------------------------ building blocks
    def vision_embed(self, br: str, patches, px, py):
        cfg, p = self.cfg, self.p
        m2 = cfg.merge_size ** 2
        a1 = gemm.gemm_nt(patches, p[f"vision_{br}.patch_w"], residual=p[f"vision_{br}.patch_b"])
        fused.gelu_fwd(a1, a1)
        r1 = fused.rope2d(a1, torch.empty_like(a1), px, py, self.inv_v)
        return gemm.gemm_nt(r1.view(r1.shape[0] // m2, m2 * cfg.vision_hidden), p[f"vision_{br}.merge_w"],
                            residual=p[f"vision_{br}.merge_b"])

    def scalar_embed(self, name, t):
        p = self.p
        s = oracle.sinusoid(t, self.cfg.timestep_freq_dim).to(torch.bfloat16)
        h = torch.nn.functional.silu(gemm.gemm_nt(s, p[name + ".w1"], residual=p[name + ".b1"]))
        return gemm.gemm_nt(h, p[name + ".w2"], residual=p[name + ".b2"])

    def alloc_cache(self, kv_rows: int):
        cfg = self.cfg
        if self.kc and self.kc[0].shape[0] >= kv_rows:
            return
        if self.sp is not None:
            from ..parallel.symm import SymmetricBuffer
            n = cfg.num_layers * kv_rows * cfg.kv_dim
            self.sp["k"] = SymmetricBuffer(n, torch.bfloat16, self.dev, self.sp["group"])
            self.sp["v"] = SymmetricBuffer(n, torch.bfloat16, self.dev, self.sp["group"])
            self.sp["rows"] = kv_rows
            shape = (cfg.num_layers, kv_rows, cfg.num_kv_heads, 128)
            self.kc = list(self.sp["k"].tensor.view(shape).unbind(0))
            self.vc = list(self.sp["v"].tensor.view(shape).unbind(0))
            return
        self.kc = [torch.zeros(kv_rows, cfg.num_kv_heads, 128, dtype=torch.bfloat16, device=self.dev)
                   for _ in range(cfg.num_layers)]
        self.vc = [torch.zeros(kv_rows, cfg.num_kv_heads, 128, dtype=torch.bfloat16, device=self.dev)
                   for _ in range(cfg.num_layers)]

    def layers(self, x, branch: int, pos3, plan, kv_rows, kv_len: int, publish=None):
        """Runs the decoder stack on rows ``x`` [R,H] with one branch's weights.  The rows'
        K/V are written to cache rows ``kv_rows`` (int64 [R]); attention reads cache rows
        [0, kv_len).  Returns the final hidden state (before the final norm).

        ``publish`` (sequence-parallel sampling): runs of rows [(first row of x, count, first cache row)]
        whose K/V go to every rank of the sequence-parallel group instead of the local cache only."""
        cfg, p, ws = self.cfg, self.p, self.ws
        R, H = x.shape
        qd, kd = cfg.q_dim, cfg.kv_dim
        if self.offload is not None:
            self.offload.set_phase("prefix" if branch == UND else "denoise")
        for l in range(cfg.num_layers):
            s = f"layers.{l}."
            if self.offload is not None:
                lw = self.offload.layer_weights(l)          # this branch's tensors, on the device
                W = WE = lambda n: lw[n]
            else:
                W = lambda n: p[s + n][branch]
                WE = lambda n: p[s + n]                     # expert mixtures are whole tensors of one branch
            h1 = fused.rmsnorm_fwd(x, W("attn_norm"), None, ws.get("i.h1", (R, H)), None, cfg.rms_eps)
            qkv = gemm.gemm_nt(h1, W("wqkv"), out=ws.get("i.qkv", (R, qd + 2 * kd)))
            qk = ws.get("i.qk", (R, qd + kd))
            fused.qknorm_rope_fwd(qkv, qk, W("qk_norm"), None, pos3, self.inv_t, self.inv_hw,
                                  cfg.num_heads, cfg.num_kv_heads, cfg.rms_eps)
            if publish is None:
                self.kc[l].view(-1, kd).index_copy_(0, kv_rows, qk[:, qd:])
                self.vc[l].view(-1, kd).index_copy_(0, kv_rows, qkv[:, qd + kd:])
            else:
                from ..parallel.symm import peer_put
                kt, vt = ws.get("i.kt", (R, kd)), ws.get("i.vt", (R, kd))
                kt.copy_(qk[:, qd:])
                vt.copy_(qkv[:, qd + kd:])
                base = l * self.sp["rows"]
                for a, n, c in publish:
                    peer_put(kt[a:a + n], self.sp["k"], (base + c) * kd)
                    peer_put(vt[a:a + n], self.sp["v"], (base + c) * kd)
                # every peer's slice of this layer is in my cache after the barrier; a peer can only come
                # back to this layer (next step) after the barriers of all later layers, i.e. after I read
                self.sp["bar"].barrier()
            q = qk[:, :qd].unflatten(1, (cfg.num_heads, 128))
            o, _ = attn_ops.attention_fwd(q, self.kc[l][:kv_len], self.vc[l][:kv_len], plan, self.scale,
                                          out=ws.get("i.o", (R, cfg.num_heads, 128)),
                                          lse=ws.get("i.lse", (cfg.num_heads, R), torch.float32))
            x1 = gemm.gemm_nt(o.view(R, qd), W("wo"), out=ws.get("i.x1", (R, H)), residual=x)
            h2 = fused.rmsnorm_fwd(x1, W("ffn_norm"), None, ws.get("i.h2", (R, H)), None, cfg.rms_eps)
            xo = ws.get(f"i.x{l & 1}", (R, H))
            if not cfg.is_moe:
                gu = gemm.gemm_nt(h2, W("w13"), out=ws.get("i.gu", (R, 2 * cfg.ffn_size)))
                act = fused.swiglu_fwd(gu, ws.get("i.act", (R, cfg.ffn_size)))
                x = gemm.gemm_nt(act, W("w2"), out=xo, residual=x1)
            else:
                x = self._moe_ffn(WE, h2, x1, branch, xo)
        return x

    def _moe_ffn(self, W, h2, x1, branch, out):
        """Dropless top-k expert FFN of one branch: device-side routing, tokens gathered into expert
        segments, one grouped GEMM per projection, weighted combine + residual (the reference loops
        over experts in Python: src/sensenova_u1/models/neo_unify/modeling_qwen3_moe.py:51-119)."""
        from ..ops import moe
        cfg, p, ws = self.cfg, self.p, self.ws
        br = "und" if branch == UND else "gen"
        K = cfg.num_experts_per_tok if branch == UND else cfg.gen_num_experts_per_tok
        R, H = h2.shape
        Fe = cfg.moe_intermediate_size
        gate = W(f"moe_{br}.gate")
        logits = gemm.gemm_nt(h2, gate, out=ws.get("i.moe.logits", (R, gate.shape[0]), torch.float32),
                              out_mode=gemm.OUT_F32_STORE)
        r = moe.route(logits, K, cfg.norm_topk_prob)
        xp = ws.get("i.moe.xp", (r.max_rows, H), zero=True)
        moe.gather(h2, r, xp)
        gu = gemm.gemm_nt(xp, W(f"moe_{br}.w13"), out=ws.get("i.moe.gu", (r.max_rows, 2 * Fe)), tile_group=r.tile_group)
        act = fused.swiglu_fwd(gu, ws.get("i.moe.act", (r.max_rows, Fe)))
        yp = gemm.gemm_nt(act, W(f"moe_{br}.w2"), out=ws.get("i.moe.yp", (r.max_rows, H)), tile_group=r.tile_group)
        return moe.combine(yp, r, x1, out)

    def final_norm(self, x, branch):
        return fused.rmsnorm_fwd(x, self.p["final_norm"][branch], None, torch.empty_like(x), None, self.cfg.rms_eps)

    # ------------------------------------------------------------------- prefix
    def prefill(self, docs_ids: Sequence[torch.Tensor], reserve_image_tokens: int,
                docs_embeds: Optional[Sequence[torch.Tensor]] = None,
                docs_pos3: Optional[Sequence[torch.Tensor]] = None):
        """Understanding-branch forward of several prompts packed as documents; fills the KV
        cache.  Returns (layouts, last hidden rows [n_docs,H]).  ``docs_embeds`` / ``docs_pos3``
        override token embeddings / (t,h,w) indexes (prompts that contain images)."""
        cfg = self.cfg
        n_docs = len(docs_ids)
        lens = [int(d.numel()) for d in docs_ids]
        layouts, kv_pos = [], 0
        for n in lens:
            layouts.append(DocLayout(kv_pos, n, kv_pos + n, n))
            kv_pos += n + reserve_image_tokens
        self.alloc_cache(_pad128(kv_pos))
        R = sum(lens)
        ids = torch.cat([d.to(self.dev) for d in docs_ids]).long()
        x = self.p["embed_tokens"].index_select(0, ids) if docs_embeds is None else torch.cat(list(docs_embeds))
        doc = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(lens)]).to(self.dev)
        if docs_pos3 is None:
            pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens]).to(self.dev)
            pos3 = torch.stack([pos, torch.zeros_like(pos), torch.zeros_like(pos)]).contiguous()
            img = None
        else:
            pos3 = torch.cat(list(docs_pos3), dim=1).to(self.dev).int().contiguous()
            pos = pos3[0]
            # tokens that share a t index with a neighbour belong to one image: bidirectional
            img = ((pos3[1] > 0) | (pos3[2] > 0) | (torch.roll(pos, 1) == pos) | (torch.roll(pos, -1) == pos)).int() * (pos + 1)
        kv_rows = torch.cat([torch.arange(lay.kv_start, lay.kv_start + n) for lay, n in zip(layouts, lens)]).to(self.dev)
        # keys: cache rows [0, kv_pos); rows not written yet are blocked
        mk = torch.zeros(kv_pos, 4, dtype=torch.int32, device=self.dev)
        mk[:, 0] = -7
        mk[:, 3] = attn_ops.FLAG_BLOCKED
        mq = attn_ops.make_meta(doc, pos, img)
        mk[kv_rows] = mq
        plan = attn_ops.build_plan(mq, mk.contiguous())
        x = self.layers(x.contiguous(), UND, pos3, plan, kv_rows, kv_pos)
        last = torch.tensor([sum(lens[:i + 1]) - 1 for i in range(n_docs)], device=self.dev)
        self._meta_k = mk
        for lay, n in zip(layouts, lens):
            lay.next_pos = int(pos3[0][sum(lens[:layouts.index(lay)]) + n - 1]) + 1
        return layouts, x.index_select(0, last)

    # ------------------------------------------------------------ text decoding
    def decode_greedy(self, layouts: List[DocLayout], last_hidden, max_new_tokens: int,
                      stop_ids: Sequence[int] = (), use_graph: bool = True, check_every: int = 8):
        """Greedy continuation: :meth:`decode` without sampling."""
        return self.decode(layouts, last_hidden, max_new_tokens, stop_ids, use_graph, check_every, sampling=None)

    @staticmethod
    def _pick_token(logits, sampling, seen=None):
        """Next token per row from fp32 logits.  ``sampling`` None: argmax.  Otherwise, in the order of transformers'
        logits processors: repetition penalty on the tokens marked in ``seen`` ([rows, vocab] bool: prompt and
        generated tokens; positive logits divided by the penalty, negative ones multiplied), then, with ``do_sample``,
        temperature, top-k and nucleus (top-p) filtering and a draw by the exponential-race form of categorical
        sampling (argmax of p / Exp(1)), which stays on the device and is capturable in a CUDA graph."""
        if not sampling:
            return logits.argmax(-1)
        lg = logits.float()
        rp = float(sampling.get("repetition_penalty", 1.0) or 1.0)
        if seen is not None and rp != 1.0:
            lg = torch.where(seen, torch.where(lg > 0, lg / rp, lg * rp), lg)
        if not sampling.get("do_sample", False):
            return lg.argmax(-1)
        t = float(sampling.get("temperature", 1.0) or 1.0)
        if t != 1.0:
            lg = lg / t
        k = int(sampling.get("top_k", 0) or 0)
        if 0 < k < lg.shape[-1]:
            kth = torch.topk(lg, k, dim=-1).values[..., -1:]
            lg = lg.masked_fill(lg < kth, float("-inf"))
        p_ = float(sampling.get("top_p", 1.0) or 1.0)
        if p_ < 1.0:
            srt, idx = torch.sort(lg, dim=-1, descending=True)
            cum = torch.softmax(srt, dim=-1).cumsum(-1)
            drop = (cum - torch.softmax(srt, dim=-1)) > p_          # keep the token that crosses the threshold
            srt = srt.masked_fill(drop, float("-inf"))
            lg = torch.full_like(lg, float("-inf")).scatter(-1, idx, srt)
        probs = torch.softmax(lg, dim=-1)
        return (probs / torch.empty_like(probs).exponential_(1.0)).argmax(-1)

    def decode(self, layouts: List[DocLayout], last_hidden, max_new_tokens: int, stop_ids: Sequence[int] = (),
               use_graph: bool = True, check_every: int = 8, sampling: Optional[dict] = None,
               prompt_ids: Optional[Sequence[torch.Tensor]] = None):
        """Continuation of every document (understanding branch), one token per step: greedy, or sampled with
        ``sampling = {do_sample, temperature, top_k, top_p, repetition_penalty, seed}`` (the knobs of the reference's
        ``generate``, src/sensenova_u1/models/neo_unify/modeling_neo_chat.py:1916-1975, examples/vqa/inference.py:29-112).
        ``prompt_ids`` (one id tensor per document) lets the repetition penalty see the prompt as well.
        The reserved image rows of the cache are used for the new tokens.

        One decode step (LM head, argmax, embedding, metadata + tile plan of the new row, 42 layers)
        is about 500 small launches and launch-bound, so after one eager step the step is captured
        in a CUDA graph and replayed; all of its state (token, position, cache row, output slot)
        lives in device tensors that the graph itself advances.  The host only looks at the tokens
        every ``check_every`` steps to see whether every document has stopped."""
        n_docs = len(layouts)
        if max_new_tokens <= 0:
            return [[] for _ in range(n_docs)]
        dev = self.dev
        st = {
            "h": last_hidden.contiguous().clone(),
            "out": torch.full((n_docs, max_new_tokens), -1, dtype=torch.long, device=dev),
            "step": torch.zeros(1, dtype=torch.long, device=dev),
            "pos": torch.tensor([lay.next_pos for lay in layouts], dtype=torch.int32, device=dev),
            "kv_rows": torch.tensor([lay.img_start for lay in layouts], dtype=torch.long, device=dev),
            "doc": torch.arange(n_docs, dtype=torch.int32, device=dev),
        }
        kv_len = self._meta_k.shape[0]
        if sampling and float(sampling.get("repetition_penalty", 1.0) or 1.0) != 1.0:
            vocab = self.p["lm_head"].shape[0]
            st["seen"] = torch.zeros(n_docs, vocab, dtype=torch.bool, device=dev)      # advanced inside the graph
            for d, ids in enumerate(prompt_ids or ()):
                st["seen"][d, ids.to(dev).long().clamp_(0, vocab - 1)] = True

        def step_fn():
            logits = gemm.gemm_nt(self.final_norm(st["h"], UND), self.p["lm_head"], out_mode=gemm.OUT_F32_STORE)
            nxt = self._pick_token(logits, sampling, st.get("seen"))
            if "seen" in st:
                st["seen"].scatter_(1, nxt.view(-1, 1), True)
            st["out"].index_copy_(1, st["step"], nxt.view(-1, 1))
            x = self.p["embed_tokens"].index_select(0, nxt)
            zero = torch.zeros_like(st["pos"])
            pos3 = torch.stack([st["pos"], zero, zero]).contiguous()
            mq = attn_ops.make_meta(st["doc"], st["pos"])
            self._meta_k.index_copy_(0, st["kv_rows"], mq)
            plan = attn_ops.build_plan(mq, self._meta_k)
            h = self.layers(x.contiguous(), UND, pos3, plan, st["kv_rows"], kv_len)
            st["h"].copy_(h)
            st["pos"].add_(1)
            st["kv_rows"].add_(1)
            st["step"].add_(1)

        done = 0
        graph = None
        stops = set(int(t) for t in stop_ids)

        def finished():
            toks = st["out"][:, :done].tolist()
            return all(any(t in stops for t in row) for row in toks) if stops else False

        if sampling and sampling.get("do_sample", False) and sampling.get("seed") is not None and dev.type == "cuda":
            torch.cuda.manual_seed(int(sampling["seed"]))
        step_fn()                                   # eager: also warms every lazy initialisation
        done = 1
        if use_graph and max_new_tokens > 2:
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step_fn()
        while done < max_new_tokens:
            if done % check_every == 0 and finished():
                break
            if graph is not None:
                graph.replay()
            else:
                step_fn()
            done += 1
        toks = st["out"][:, :done].tolist()
        out = []
        for row in toks:
            cut = len(row)
            for i, t in enumerate(row):
                if t in stops:
                    cut = i + 1
                    break
            out.append(row[:cut])
        for lay in layouts:                         # every executed step consumed one cache row
            lay.img_start += done
            lay.prefix_len += done
            lay.next_pos += done
        self.last_decode_steps, self.last_decode_graph = done, graph is not None
        return out

    # --------------------------------------------------------------- generation
    @torch.no_grad()
    def t2i(self, cond_ids: torch.Tensor, uncond_ids: Optional[torch.Tensor], image_size=(256, 256),
            num_steps: int = 50, cfg_scale: float = 4.0, timestep_shift: float = 3.0,
            cfg_norm: str = "none", cfg_interval=(0.0, 1.0), t_eps: float = 0.02, seed: int = 0,
            batch_size: int = 1, noise: Optional[torch.Tensor] = None, cfg_group=None, par_group=None):
        """Text-to-image: returns pixels [B,3,H,W] float32 in [-1,1].  ``image_size`` = (W,H).
        ``cfg_group``: two ranks, one per guidance branch; ``par_group``: all ranks of a guidance-parallel x
        sequence-parallel run (see :meth:`denoise`)."""
        use_cfg = cfg_scale > 1 and uncond_ids is not None
        branches = [(cond_ids, None, None)] + ([(uncond_ids, None, None)] if use_cfg else [])
        return self.denoise([branches] * batch_size, image_size, num_steps, cfg_scale, 0.0, timestep_shift,
                            cfg_norm, cfg_interval, t_eps, seed, noise, cfg_group=cfg_group if use_cfg else None,
                            par_group=par_group)

    def _cfg_parallel(self, group, nb: int, numel: int, par_group=None):
        """Exchange state of parallel sampling: two symmetric prediction buffers ([branches][B*T][token_dim])
        and a flag barrier over ``par_group``, the ranks that exchange predictions (default: ``group``)."""
        import torch.distributed as dist
        from ..parallel.symm import FlagBarrier, SymmetricBuffer
        if group is not None and dist.get_world_size(group) != nb:
            raise ValueError(f"guidance-parallel sampling needs one rank per branch ({nb}), "
                             f"group has {dist.get_world_size(group)}")
        par_group = par_group if par_group is not None else group
        st = getattr(self, "_cfgpar", None)
        if st is None or st["numel"] < numel or st["nb"] != nb or st["group"] is not par_group:
            st = {"numel": numel, "nb": nb, "rank": dist.get_rank(group) if group is not None else None,
                  "group": par_group, "bar": FlagBarrier(par_group, self.dev),
                  "x": [SymmetricBuffer(nb * numel, torch.bfloat16, self.dev, par_group) for _ in range(2)]}
            self._cfgpar = st
        return st

    @torch.no_grad()
    def denoise(self, samples, image_size=(256, 256), num_steps: int = 50, cfg_scale: float = 4.0,
                img_cfg_scale: float = 1.0, timestep_shift: float = 3.0, cfg_norm: str = "none",
                cfg_interval=(0.0, 1.0), t_eps: float = 0.02, seed: int = 0, noise: Optional[torch.Tensor] = None,
                cfg_group=None, par_group=None):
        """Flow-matching Euler sampling of one image per sample.

        Sequence-parallel sampling (after :meth:`enable_sequence_parallel`): every rank of the group runs the
        decoder on its contiguous slice of each image's tokens; keys / values are exchanged per layer, the
        predictions per step, through peer memory.  Combines with ``cfg_group`` (ranks = branches x slices;
        ``par_group`` is then the group of all of them, default the world group).

        ``cfg_group``: guidance-parallel sampling.  A process group with one rank per guidance branch
        (2 for text-to-image, 3 for editing): rank r runs branch r only, stores its prediction into
        every rank's symmetric buffer with peer stores, and after a device-side flag barrier every
        rank applies the same fused guidance + Euler step, so the latents stay bit-identical without a
        broadcast.  The reference has no multi-GPU sampler (docs/inference_infra.md:20-21 points to
        an external engine for CFG/SP parallelism).

        ``samples[b]`` lists the guidance branches of sample b as (ids, embeds or None, pos3 or None):
        branch 0 the full condition, branch 1 the unconditional prompt, branch 2 (editing /
        interleaved generation) the image-only condition; v = v_u + s_t (v_c - v_i) + s_i (v_i - v_u)
        (modeling_neo_chat.py:1606-1663).  Every branch of every sample is one document of the same
        packed forward.  Returns pixels [B,3,H,W] in [-1,1]."""
        cfg = self.cfg
        W, Hh = image_size
        tp = cfg.token_pixels
        th, tw = Hh // tp, W // tp
        T = th * tw
        batch_size = len(samples)
        nb = len(samples[0])
        par = None
        sp = self.sp
        if sp is not None and (T % (128 * sp["world"]) != 0):
            raise ValueError(f"sequence-parallel sampling needs the image token count ({T}) to be a multiple of "
                             f"128 x {sp['world']} ranks")
        use_cfg_par = cfg_group is not None and nb > 1
        if use_cfg_par or sp is not None:
            import torch.distributed as dist
            if use_cfg_par and sp is not None and par_group is None:
                par_group = dist.group.WORLD
            par = self._cfg_parallel(cfg_group if use_cfg_par else None, nb, batch_size * T * cfg.token_dim,
                                     par_group if par_group is not None else (cfg_group if use_cfg_par else sp["group"]))
            if use_cfg_par:
                samples = [[smp[par["rank"]]] for smp in samples]       # my guidance branch only
        nb_all, nb = nb, len(samples[0])
        Tl = T // sp["world"] if sp is not None else T                   # image tokens of one document on this rank
        s0 = sp["rank"] * Tl if sp is not None else 0
        prompts = [br for smp in samples for br in smp]
        has_emb = any(e is not None for _, e, _ in prompts)
        layouts, _ = self.prefill([p[0] for p in prompts], reserve_image_tokens=T,
                                  docs_embeds=[p[1] if p[1] is not None else self.p["embed_tokens"].index_select(
                                      0, p[0].to(self.dev).long()) for p in prompts] if has_emb else None,
                                  docs_pos3=[p[2] if p[2] is not None else torch.stack(
                                      [torch.arange(p[0].numel()), torch.zeros(p[0].numel(), dtype=torch.long),
                                       torch.zeros(p[0].numel(), dtype=torch.long)]) for p in prompts] if has_emb else None)
        n_docs = len(prompts)
        hh = torch.arange(th, dtype=torch.int32).view(th, 1).expand(th, tw).reshape(-1)
        ww = torch.arange(tw, dtype=torch.int32).view(1, tw).expand(th, tw).reshape(-1)
        # rows are grouped by branch: [all conditional images | all unconditional | all image-only]
        order = [i for k in range(nb) for i in range(n_docs) if i % nb == k]
        pos3 = torch.cat([torch.stack([torch.full((T,), layouts[i].next_pos, dtype=torch.int32), hh, ww]) for i in order],
                         dim=1).to(self.dev).contiguous()
        kv_rows = torch.cat([torch.arange(layouts[i].img_start, layouts[i].img_start + T) for i in order]).to(self.dev)
        doc = torch.cat([torch.full((T,), i, dtype=torch.int32) for i in order]).to(self.dev)
        big = torch.full_like(doc, 1 << 28)
        mq = attn_ops.make_meta(doc, big)
        mk = self._meta_k.clone()
        mk[kv_rows] = attn_ops.make_meta(doc, torch.zeros_like(doc))
        publish = None
        if sp is not None:
            # my rows: the slice [s0, s0 + Tl) of every document, in the same document order
            loc = torch.cat([torch.arange(j * T + s0, j * T + s0 + Tl) for j in range(len(order))]).to(self.dev)
            pos3 = pos3.index_select(1, loc).contiguous()
            kv_rows = kv_rows.index_select(0, loc)
            mq = mq.index_select(0, loc).contiguous()
            publish = [(j * Tl, Tl, layouts[i].img_start + s0) for j, i in enumerate(order)]
        plan = attn_ops.build_plan(mq, mk.contiguous())
        kv_len = mk.shape[0]
        ns = min(math.sqrt(T / float(cfg.noise_scale_base_image_seq_len)) * cfg.noise_scale
                 if cfg.noise_scale_mode in ("resolution", "dynamic", "dynamic_sqrt") else cfg.noise_scale,
                 cfg.noise_scale_max_value)
        if noise is None:
            g = torch.Generator(device=self.dev).manual_seed(seed)
            noise = torch.randn(batch_size, 3, Hh, W, device=self.dev, generator=g)
        img = ns * noise.float()
        z = img.reshape(batch_size, 3, th, tp, tw, tp).permute(0, 2, 4, 3, 5, 1).reshape(batch_size * T, cfg.token_dim).contiguous()
        m, ps = cfg.merge_size, cfg.patch_size
        patches = z.reshape(batch_size * T, m, ps, m, ps, 3).permute(0, 1, 3, 5, 2, 4).reshape(
            batch_size * T * m * m, cfg.patch_dim).to(torch.bfloat16).contiguous()
        ty = hh.view(-1, 1, 1) * m + torch.arange(m, dtype=torch.int32).view(1, m, 1)
        tx = ww.view(-1, 1, 1) * m + torch.arange(m, dtype=torch.int32).view(1, 1, m)
        py = ty.expand(T, m, m).reshape(-1).repeat(batch_size).to(self.dev).contiguous()
        px = tx.expand(T, m, m).reshape(-1).repeat(batch_size).to(self.dev).contiguous()
        ts = torch.linspace(0.0, 1.0, num_steps + 1)
        ts = apply_time_schedule(ts, T, cfg, timestep_shift=timestep_shift).tolist()
        ns_emb = None
        if cfg.add_noise_scale_embedding:
            ns_emb = self.scalar_embed("noise_scale_embedder", torch.full((1,), ns / cfg.noise_scale_max_value, device=self.dev))
        BT = batch_size * T
        BTl = batch_size * Tl
        m2 = m * m
        if sp is not None:
            prow = torch.cat([torch.arange((b * T + s0) * m2, (b * T + s0 + Tl) * m2) for b in range(batch_size)]).to(self.dev)
            px_l, py_l = px.index_select(0, prow).contiguous(), py.index_select(0, prow).contiguous()
        plan_c = None
        for step in range(num_steps):
            t, t_next = ts[step], ts[step + 1]
            if sp is not None:
                emb = self.vision_embed("gen", patches.index_select(0, prow), px_l, py_l)
            else:
                emb = self.vision_embed("gen", patches, px, py)
            e_t = self.scalar_embed("timestep_embedder", torch.full((1,), t, device=self.dev))
            emb = emb + (e_t + ns_emb if ns_emb is not None else e_t)
            in_interval = cfg_interval[0] <= t <= cfg_interval[1]
            branches = nb if (nb > 1 and in_interval) else 1
            if use_cfg_par:
                branches = nb_all if in_interval else 1
            if branches == nb or use_cfg_par:
                x = emb if nb == 1 else torch.cat([emb] * nb, 0)
                h = self.layers(x.contiguous(), GEN, pos3, plan, kv_rows, kv_len, publish)
            else:  # outside the guidance interval only the conditional documents run
                sub = slice(0, BTl)
                if plan_c is None:
                    plan_c = attn_ops.build_plan(mq[sub].contiguous(), mk.contiguous())
                h = self.layers(emb.contiguous(), GEN, pos3[:, sub].contiguous(), plan_c, kv_rows[sub], kv_len,
                                publish[:batch_size] if publish is not None else None)
            hf = self.final_norm(h, GEN)
            if cfg.use_pixel_head:
                # convolutional decoder: cuDNN convolutions on the token grids (not a tcgen05 path)
                x_pred = oracle.pixel_head(self.p, hf, [(th, tw)] * (hf.shape[0] // T), cfg).to(torch.bfloat16).contiguous()
            else:
                a1 = gemm.gemm_nt(hf, self.p["fm_head.w1"], residual=self.p["fm_head.b1"])
                fused.gelu_fwd(a1, a1)
                x_pred = gemm.gemm_nt(a1, self.p["fm_head.w2"], residual=self.p["fm_head.b2"])
            if par is not None:
                from ..parallel.symm import peer_put
                buf = par["x"][step & 1]                     # two buffers: a slow peer may still read the other
                if sp is None:
                    peer_put(x_pred, buf, par["rank"] * BT * cfg.token_dim)
                else:
                    # my token slice of every (branch, sample) goes to its place in every rank's buffer
                    for k in range(x_pred.shape[0] // BTl):
                        kb = par["rank"] if use_cfg_par else k
                        for b in range(batch_size):
                            peer_put(x_pred[(k * batch_size + b) * Tl:(k * batch_size + b + 1) * Tl], buf,
                                     ((kb * batch_size + b) * T + s0) * cfg.token_dim)
                par["bar"].barrier()
                x_pred = buf.tensor
            _lib.call("sampler_step", c_void_p(x_pred.data_ptr()), c_void_p(z.data_ptr()),
                      c_void_p(patches.data_ptr()), c_void_p(self.stats.data_ptr()), c_int(BT),
                      c_int(cfg.token_dim), c_int(branches), c_int(ps), c_int(m), c_float(t), c_float(t_next),
                      c_float(t_eps), c_float(cfg_scale), c_float(img_cfg_scale), c_int(1 if branches > 1 else 0),
                      c_int(CFG_NORMS[cfg_norm]), c_int(1 if step == 0 else 0), c_void_p(_lib.stream()))
        self.last_layouts = layouts
        return z.reshape(batch_size, th, tw, tp, tp, 3).permute(0, 5, 1, 3, 2, 4).reshape(batch_size, 3, Hh, W)
