"""ZeRO-1 AdamW over the flat parameter arenas.

Each data-parallel rank owns one contiguous range of every arena: it receives the
sum of the gradients of that range (reduce-scatter), updates the fp32 master of the
range with the fused unscale + clip + AdamW kernel, and the updated bf16 weights are
all-gathered back in place.  This is the reduce-scatter / all-gather form of the
reference's ZeRO-1, which all-reduces full gradients and then broadcasts every
partition (training/sensenovalm/solver/optimizer/hybrid_zero_optim.py:626-690,
832-1070) at twice the wire traffic; the update itself is numerically the same.

On CPU tensors (gloo tests) the same schedule runs with a PyTorch AdamW on an fp32
master of the shard.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..models.params import ParamStore


@dataclass
class AdamConfig:
    lr: float = 2e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.0
    clip_grad_norm: float = 1.0
    state_dtype: str = "auto"      # "fp32" | "bf16" | "auto" (fp32 when it fits in device memory)
    lr_scale: Optional[Dict[str, float]] = None   # per role: vit, llm, fm_modules, embed, ...; "mot_gen": generation branch
    frozen: Optional[Dict[str, List[Tuple[int, int]]]] = None   # train.freeze.frozen_ranges: never updated


class ZeroAdamW:
    """Bucketed ZeRO-1.  Every bucket of an arena (see ``ParamStore.buckets``) is split evenly
    over the ranks; rank r owns piece r of every bucket.  A bucket's gradients can be
    reduce-scattered as soon as its backward is done (``reduce_bucket``), while the rest of
    the backward pass still runs; after the step each bucket's weights are all-gathered
    asynchronously and ``wait_bucket`` is called before the next forward touches them."""

    def __init__(self, store: ParamStore, cfg: AdamConfig, group=None, grad_divisor: float = 1.0):
        self.store, self.cfg, self.group = store, cfg, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.grad_divisor = grad_divisor
        self.step_count = 0
        self.dev = store.device
        self.cuda = self.dev.type == "cuda"
        self.lr = cfg.lr
        # pieces[arena] = list of (bucket name, bucket lo, bucket hi, my lo, my hi, state offset)
        self.pieces: Dict[str, List[Tuple[str, int, int, int, int, int]]] = {}
        self.state: Dict[str, Dict[str, torch.Tensor]] = {}
        total_own = 0
        # arenas whose content differs per rank (expert-parallel weights): updated whole, never
        # reduced or gathered; their gradient norm still joins the global norm
        self.local_arenas = {a for a in store.sizes if a == "exp"}
        for a in store.sizes:
            lst, off = [], 0
            aw, ar = (1, 0) if a in self.local_arenas else (self.world, self.rank)
            for name, lo, hi in store.buckets(a):
                if (hi - lo) % (aw * 8):
                    raise ValueError(f"bucket {name} of arena {a} ({hi - lo}) does not split over {aw} ranks")
                per = (hi - lo) // aw
                lst.append((name, lo, hi, lo + ar * per, lo + (ar + 1) * per, off))
                off += per
            self.pieces[a] = lst
            total_own += off
        sd = cfg.state_dtype
        if sd == "auto":
            sd = "fp32"
            if self.cuda:
                free, _ = torch.cuda.mem_get_info(self.dev)
                need = total_own * (2 + 8) + (14 << 30)
                if need > free:
                    sd = "bf16"
        self.state_dtype = torch.float32 if sd == "fp32" else torch.bfloat16
        for a, lst in self.pieces.items():
            n = sum(p[4] - p[3] for p in lst)
            st = {"m": torch.zeros(n, dtype=self.state_dtype, device=self.dev),
                  "v": torch.zeros(n, dtype=self.state_dtype, device=self.dev)}
            if self.cuda:
                st["lo"] = torch.zeros(n, dtype=torch.int16, device=self.dev)
            else:
                st["master"] = torch.cat([store.arena[a][p[3]:p[4]].float() for p in lst]) if lst else \
                    torch.zeros(0)
            self.state[a] = st
        self.norm_sq = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self.skipped = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.runs = {a: self._runs(a) for a in store.sizes}
        self._reduced = set()
        self._rs_work: List = []
        self._ag_work: Dict[Tuple[str, str], object] = {}
        # legacy view: first / last owned element of each arena (tests, checkpoints)
        self.shard = {a: (lst[0][3], lst[-1][4]) for a, lst in self.pieces.items()}

    def _runs(self, arena) -> List[Tuple[int, int, float, float]]:
        """Merged (start, end, lr_scale, weight_decay) runs over the whole arena."""
        scales = self.cfg.lr_scale or {}
        gen_sc = float(scales.get("mot_gen", 1.0))     # extra factor on the generation branch's weights
        runs: List[List] = []
        pos = 0
        for s, e, spec in self.store.segments(arena):
            wd = self.cfg.weight_decay if spec.decay else 0.0
            sc = scales.get(spec.role, 1.0)
            pieces = [(e, sc)]
            if gen_sc != 1.0:
                if ".moe_gen." in spec.name or spec.name.startswith(("vision_gen.", "fm_head.", "timestep_embedder.",
                                                                     "noise_scale_embedder.")):
                    pieces = [(e, sc * gen_sc)]
                elif len(spec.shape) > 1 and spec.shape[0] == 2 and spec.name.startswith(("layers.", "mtp.", "final_norm")):
                    # dual tensor [understanding | generation]: the second half is the generation branch
                    pieces = [(s + (e - s) // 2, sc), (e, sc * gen_sc)]
            for end, psc in pieces:
                if runs and runs[-1][2] == psc and runs[-1][3] == wd:
                    runs[-1][1] = end
                else:
                    runs.append([pos, end, psc, wd])   # the alignment gap before a tensor joins its run
                pos = end
        if runs:
            runs[-1][1] = self.store.sizes[arena]
        frozen = (self.cfg.frozen or {}).get(arena) or []
        if frozen:
            # cut the runs at the frozen ranges; inside them learning rate and decay are 0
            cut: List[List] = []
            for s, e, sc, wd in runs:
                pos = s
                for fs, fe in frozen:
                    a, b = max(fs, s), min(fe, e)
                    if b <= a:
                        continue
                    if a > pos:
                        cut.append([pos, a, sc, wd])
                    cut.append([a, b, 0.0, 0.0])
                    pos = b
                if pos < e:
                    cut.append([pos, e, sc, wd])
            runs = cut
        return [tuple(r) for r in runs]

    def own_ranges(self, arena):
        """(start, end, lr_scale, weight_decay, state offset) pieces this rank updates."""
        out = []
        for _, _, _, mlo, mhi, soff in self.pieces[arena]:
            for s, e, sc, wd in self.runs[arena]:
                s2, e2 = max(s, mlo), min(e, mhi)
                if e2 > s2:
                    out.append((s2, e2, sc, wd, soff + (s2 - mlo)))
        return out

    # -------------------------------------------------------------- gradients
    def reduce_bucket(self, arena: str, name: str) -> None:
        """Starts the reduce-scatter of one bucket (asynchronous on NCCL's stream)."""
        if self.world == 1 or (arena, name) in self._reduced or arena in self.local_arenas:
            return
        for bname, lo, hi, mlo, mhi, _ in self.pieces[arena]:
            if bname != name:
                continue
            g = self.store.grad_arena[arena]
            if self.cuda:
                w = dist.reduce_scatter_tensor(g[mlo:mhi], g[lo:hi], op=dist.ReduceOp.SUM, group=self.group,
                                               async_op=True)
                self._rs_work.append(w)
            else:
                dist.all_reduce(g[lo:hi], op=dist.ReduceOp.SUM, group=self.group)
            self._reduced.add((arena, name))

    def reduce_gradients(self):
        """Reduces every bucket that has not been reduced yet, then waits for all of them."""
        for a, lst in self.pieces.items():
            for name, *_ in lst:
                self.reduce_bucket(a, name)
        for w in self._rs_work:
            w.wait()
        self._rs_work.clear()
        self._reduced.clear()

    def grad_norm_sq(self) -> torch.Tensor:
        self.norm_sq.zero_()
        for a, lst in self.pieces.items():
            for _, _, _, mlo, mhi, _ in lst:
                g = self.store.grad_arena[a][mlo:mhi]
                if self.cuda:
                    from ..ops import fused
                    fused.sumsq(g, self.norm_sq)
                else:
                    self.norm_sq += g.float().pow(2).sum()
        if self.world > 1:
            dist.all_reduce(self.norm_sq, op=dist.ReduceOp.SUM, group=self.group)
        return self.norm_sq

    # ------------------------------------------------------------------ step
    def step(self, lr: Optional[float] = None) -> None:
        c = self.cfg
        lr = self.lr if lr is None else lr
        self.step_count += 1
        self.reduce_gradients()
        nsq = self.grad_norm_sq()
        pre = 1.0 / self.grad_divisor
        self.last_grad_norm = nsq.detach().float().sqrt() * pre      # device scalar, logged by the trainer
        if self.cuda:
            from ..ops import fused
            for a in self.pieces:
                st = self.state[a]
                P, G = self.store.arena[a], self.store.grad_arena[a]
                for s, e, sc, wd, so in self.own_ranges(a):
                    n = e - s
                    fused.adamw(P[s:e], st["lo"][so:so + n], G[s:e], st["m"][so:so + n], st["v"][so:so + n],
                                lr=lr * sc, beta1=c.beta1, beta2=c.beta2, eps=c.eps, weight_decay=wd,
                                step=self.step_count, grad_prescale=pre, norm_sq=nsq,
                                max_norm=c.clip_grad_norm, skipped=self.skipped)
        else:
            norm = float(nsq.sqrt()) * pre
            if not math.isfinite(norm):
                self.skipped += 1
            else:
                coef = min(1.0, c.clip_grad_norm / (norm + 1e-6)) if c.clip_grad_norm > 0 else 1.0
                bc1 = 1 - c.beta1 ** self.step_count
                bc2 = 1 - c.beta2 ** self.step_count
                for a in self.pieces:
                    st = self.state[a]
                    for s, e, sc, wd, so in self.own_ranges(a):
                        n = e - s
                        g = self.store.grad_arena[a][s:e].float() * (pre * coef)
                        m, v, w = st["m"][so:so + n], st["v"][so:so + n], st["master"][so:so + n]
                        m.mul_(c.beta1).add_(g, alpha=1 - c.beta1)
                        v.mul_(c.beta2).addcmul_(g, g, value=1 - c.beta2)
                        w.mul_(1 - lr * sc * wd)
                        w.addcdiv_(m.float(), (v.float().sqrt() / math.sqrt(bc2)).add_(c.eps), value=-lr * sc / bc1)
                        self.store.arena[a][s:e] = w.to(self.store.dtype)
        self.gather_params()

    def gather_params(self):
        """Starts the all-gather of every bucket's updated weights, in forward order."""
        if self.world == 1:
            return
        for a, lst in self.pieces.items():
            if a in self.local_arenas:
                continue
            P = self.store.arena[a]
            for name, lo, hi, mlo, mhi, _ in lst:
                if self.cuda:
                    self._ag_work[(a, name)] = dist.all_gather_into_tensor(P[lo:hi], P[mlo:mhi], group=self.group,
                                                                           async_op=True)
                else:
                    dist.all_gather_into_tensor(P[lo:hi], P[mlo:mhi].clone(), group=self.group)

    def wait_bucket(self, arena: str, name: str) -> None:
        w = self._ag_work.pop((arena, name), None)
        if w is not None:
            w.wait()

    def wait_all(self) -> None:
        for w in self._ag_work.values():
            w.wait()
        self._ag_work.clear()

    # ------------------------------------------------------------ checkpoint
    def state_dict(self):
        return {"step": self.step_count, "lr": self.lr, "world": self.world, "rank": self.rank,
                "pieces": {a: [(p[0], p[3], p[4]) for p in lst] for a, lst in self.pieces.items()},
                "state": {a: {k: v.cpu() for k, v in st.items()} for a, st in self.state.items()}}

    def load_state_dict(self, sd):
        if sd["world"] != self.world:
            raise ValueError(f"optimizer shards were saved with zero size {sd['world']}, now {self.world}")
        self.step_count = sd["step"]
        self.lr = sd.get("lr", self.lr)
        for a, st in sd["state"].items():
            for k, v in st.items():
                self.state[a][k].copy_(v)


class PeerZeroAdamW(ZeroAdamW):
    """ZeRO-1 whose collectives are done by this package's kernels over NVLink peer memory
    (csrc/optim.cu: zero_rs_sumsq, zero_adamw_push) instead of NCCL.  Needs the arenas in
    symmetric memory (``parallel.symm.symmetric_arenas``).  Only the scalar gradient norm
    still goes through NCCL.  Each bucket's pull starts as soon as every rank has signalled
    that bucket's backward done (flag words in symmetric memory, bounded waits), so it
    overlaps the rest of the backward pass; the weight push doubles as the all-gather."""

    def __init__(self, store: ParamStore, cfg: AdamConfig, group=None, grad_divisor: float = 1.0):
        super().__init__(store, cfg, group=group, grad_divisor=grad_divisor)
        if store.symm is None:
            raise ValueError("PeerZeroAdamW needs symmetric arenas")
        if store.grad_arena["mat"].dtype != torch.bfloat16:
            raise ValueError("peer reduce-scatter expects bf16 matrix gradients")
        from ..parallel.symm import SymmetricBuffer
        self.slots = {}
        n = 0
        for a, lst in self.pieces.items():
            if a in self.local_arenas:
                continue
            for name, *_ in lst:
                self.slots[(a, name)] = (n, n + 1)      # (gradients ready, weights ready)
                n += 2
        self.flags = SymmetricBuffer(n * self.world, torch.int32, self.dev, group)
        self.side = torch.cuda.Stream(device=self.dev)
        self._pulled = set()
        self.flags.barrier()

    def _call(self, name, *args):
        from ..ops import _lib
        _lib.call(name, *args)

    def reduce_bucket(self, arena: str, name: str) -> None:
        import ctypes
        from ..ops._lib import c_int, c_ll, c_void_p
        if (arena, name) in self._pulled or arena in self.local_arenas:
            return
        self._pulled.add((arena, name))
        if arena == "vec":
            # fp32, tiny: summed with NCCL (kept out of the bf16 peer kernel on purpose)
            dist.all_reduce(self.store.grad_arena["vec"], group=self.group)
            return
        seq = self.step_count + 1
        slot_g, _ = self.slots[(arena, name)]
        cur = torch.cuda.current_stream()
        self._call("signal_peers", self.flags.c_ptrs, c_int(self.world), c_int(self.rank), c_int(slot_g),
                   c_int(seq), c_void_p(cur.cuda_stream))
        # The pull runs on a side stream behind (1) this GPU's own backward of the bucket, ordered
        # by a stream event, and (2) the peers' signals, awaited by a ONE-warp kernel.  The pull
        # kernel itself never spins: hundreds of spinning CTAs would hold registers that the
        # attention kernels of the still-running backward need, and nothing would make progress.
        self.side.wait_stream(cur)
        self._call("wait_flags", c_void_p(self.flags.tensor.data_ptr()), c_int(self.world), c_int(slot_g),
                   c_int(seq), c_void_p(self.side.cuda_stream))
        for bname, lo, hi, mlo, mhi, _ in self.pieces[arena]:
            if bname != name:
                continue
            self._call("zero_rs_sumsq", self.store.symm["grad"][arena].c_ptrs, c_int(self.world),
                       c_int(self.rank), c_ll(mlo), c_ll(mhi - mlo), c_void_p(None),
                       c_int(slot_g), c_int(seq), c_void_p(self.norm_sq.data_ptr()),
                       c_void_p(self.side.cuda_stream))

    _pulled_first_sync = False

    def begin_step(self):
        """Call before the backward pass of the last micro-batch: clears the norm accumulator."""
        self.norm_sq.zero_()
        self._pulled.clear()
        self._pulled_first_sync = False

    def reduce_gradients(self):
        for a, lst in self.pieces.items():
            for name, *_ in lst:
                self.reduce_bucket(a, name)
        torch.cuda.current_stream().wait_stream(self.side)

    def grad_norm_sq(self) -> torch.Tensor:
        # matrix pieces were accumulated by the pull kernels; add this rank's share of the vec arena
        from ..ops import fused
        for a in ["vec"] + sorted(self.local_arenas):
            for _, _, _, mlo, mhi, _ in self.pieces[a]:
                fused.sumsq(self.store.grad_arena[a][mlo:mhi], self.norm_sq)
        dist.all_reduce(self.norm_sq, op=dist.ReduceOp.SUM, group=self.group)
        return self.norm_sq

    def step(self, lr: Optional[float] = None) -> None:
        from ..ops import fused
        from ..ops._lib import c_float, c_int, c_ll, c_void_p
        c = self.cfg
        lr = self.lr if lr is None else lr
        self.reduce_gradients()
        self.step_count += 1
        nsq = self.grad_norm_sq()
        pre = 1.0 / self.grad_divisor
        self.last_grad_norm = nsq.detach().float().sqrt() * pre      # device scalar, logged by the trainer
        bc1 = 1.0 - c.beta1 ** self.step_count
        bc2 = 1.0 - c.beta2 ** self.step_count
        st_flag = 0 if self.state_dtype == torch.bfloat16 else 1
        cur = torch.cuda.current_stream().cuda_stream
        for a in self.pieces:
            st = self.state[a]
            G = self.store.grad_arena[a]
            for s, e, sc, wd, so in self.own_ranges(a):
                n = e - s
                if a == "vec" or a in self.local_arenas:
                    fused.adamw(self.store.arena[a][s:e], st["lo"][so:so + n], G[s:e], st["m"][so:so + n],
                                st["v"][so:so + n], lr=lr * sc, beta1=c.beta1, beta2=c.beta2, eps=c.eps,
                                weight_decay=wd, step=self.step_count, grad_prescale=pre, norm_sq=nsq,
                                max_norm=c.clip_grad_norm, skipped=self.skipped)
                    continue
                self._call("zero_adamw_push", self.store.symm["arena"][a].c_ptrs, c_int(self.world),
                           c_int(self.rank), c_ll(s), c_void_p(st["lo"][so:so + n].data_ptr()),
                           c_void_p(G[s:e].data_ptr()), c_void_p(st["m"][so:so + n].data_ptr()),
                           c_void_p(st["v"][so:so + n].data_ptr()), c_ll(n), c_int(st_flag),
                           c_float(lr * sc), c_float(c.beta1), c_float(c.beta2), c_float(c.eps), c_float(wd),
                           c_float(bc1), c_float(bc2), c_float(pre), c_void_p(nsq.data_ptr()),
                           c_float(c.clip_grad_norm), c_void_p(self.skipped.data_ptr()), c_void_p(cur))
        # vec arena: small, gathered with NCCL; matrix buckets: publish "weights ready"
        for name, lo, hi, mlo, mhi, _ in self.pieces["vec"]:
            P = self.store.arena["vec"]
            dist.all_gather_into_tensor(P[lo:hi], P[mlo:mhi], group=self.group)
        for (a, name), (_, slot_w) in self.slots.items():
            if a == "mat":
                self._call("signal_peers", self.flags.c_ptrs, c_int(self.world), c_int(self.rank),
                           c_int(slot_w), c_int(self.step_count), c_void_p(cur))
        self._need_wait = {k for k in self.slots if k[0] == "mat"}

    _need_wait = set()

    def gather_params(self):
        return

    def wait_bucket(self, arena: str, name: str) -> None:
        from ..ops._lib import c_int, c_void_p
        if (arena, name) not in self._need_wait:
            return
        self._need_wait.discard((arena, name))
        _, slot_w = self.slots[(arena, name)]
        self._call("wait_flags", c_void_p(self.flags.tensor.data_ptr()), c_int(self.world), c_int(slot_w),
                   c_int(self.step_count), c_void_p(torch.cuda.current_stream().cuda_stream))

    def wait_all(self) -> None:
        for a, name in list(self._need_wait):
            self.wait_bucket(a, name)
