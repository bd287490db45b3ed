"""Pipeline (x tensor) parallel training of the CUDA engine: 1F1B or ZB-H1 over the engine's phases.

Reference: PipelineScheduler (training/sensenovalm/core/scheduler/pipeline_scheduler.py:588-869), the MoT stage
partition (sensenovavl/model/sensenovavl_moe_chat/modeling_sensenovavl_chat_mot.py:1598), p2p
(core/scheduler/comm/p2p.py:123-264).  Layout on one node: ``rank = pp_rank * tp + tp_rank``; the ranks of a stage
form a tensor-parallel group (parallel/tensor_engine.py), stage ``s`` holds the decoder layers
``partition_uniform(L, pp)[s]``, the first stage also runs the embeddings / pixel front-ends, the last the final
norm, heads and losses.  Every rank is given the same micro-batches (token metadata is needed by every stage's
attention; pixels only by the ends).  Activations ``[S, H]`` travel by NCCL point-to-point on two communicators
(see ``parallel/pipeline.py``), posted one slot ahead so that they overlap compute; inside a stage the engine
recomputes every layer in backward ("full" policy), so a micro-batch in flight holds one ``[S, H]`` tensor per local
layer.  Token embedding and LM head are separate tensors in this model family (no tied weights), so no gradient is
shared between the pipeline ends.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..config import ModelConfig
from ..data.batch import PackedBatch
from ..models.params import ParamStore
from .pipeline import PipelineStage, make_pipeline_groups, partition_uniform
from .tensor_engine import shard_store_tp, tp_local_config


def stage_store(full: ParamStore, l0: int, l1: int, **kw) -> ParamStore:
    """A store with the decoder layers ``[l0, l1)`` of ``full`` (renumbered from 0) and every non-layer tensor."""
    cfg = full.cfg.replace(num_layers=l1 - l0)
    st = ParamStore(cfg, device=full.device, dtype=full.dtype, **kw)
    for name, v in st.p.items():
        if name.startswith("layers."):
            _, l, rest = name.split(".", 2)
            v.copy_(full.p[f"layers.{l0 + int(l)}.{rest}"])
        else:
            v.copy_(full.p[name])
    return st


class PipelineTrainer:
    """``tp x pp`` ranks of one job; ``step(batches)`` runs all micro-batches through the schedule and applies the
    optimizer.  Weights come from ``init_seed`` (the full model is drawn on every rank and cut to this rank's stage
    and tensor-parallel slice, so any layout starts from the same model) or from ``full_store``."""

    def __init__(self, cfg: ModelConfig, tp: int, pp: int, device, adam=None, init_seed: int = 0, init_std: float = 0.02,
                 full_store: Optional[ParamStore] = None, schedule: str = "1f1b", max_tokens: int = 16384):
        from ..train.optimizer import AdamConfig
        from ..train.trainer import Trainer
        world, rank = dist.get_world_size(), dist.get_rank()
        if world != tp * pp:
            raise ValueError(f"{world} ranks for tp {tp} x pp {pp}")
        self.cfg, self.tp, self.pp, self.dev = cfg, tp, pp, torch.device(device)
        self.pp_rank, self.tp_rank = rank // tp, rank % tp
        # groups: every rank creates every group, in the same order
        self.tp_group = None
        for s in range(pp):
            grp = dist.new_group(list(range(s * tp, (s + 1) * tp)))
            if s == self.pp_rank:
                self.tp_group = grp
        fwd = bwd = None
        for j in range(tp):
            f, b_ = make_pipeline_groups(list(range(j, world, tp)))
            if j == self.tp_rank:
                fwd, bwd = f, b_
        l0, l1 = partition_uniform(cfg.num_layers, pp)[self.pp_rank]
        self.layers = (l0, l1)
        full = full_store
        if full is None:
            full = ParamStore(cfg, device=self.dev, with_grads=False)
            full.init_weights(init_seed, std=init_std)
        st = stage_store(full, l0, l1, with_grads=(tp == 1))
        self.store = shard_store_tp(st, tp, self.tp_rank) if tp > 1 else st
        del st, full
        if self.dev.type == "cuda":
            torch.cuda.empty_cache()
        local_cfg = tp_local_config(cfg.replace(num_layers=l1 - l0), tp)
        self.trainer = Trainer(local_cfg, self.store, adam or AdamConfig(), tp_group=self.tp_group if tp > 1 else None,
                               dp_group=self._solo_group(world, rank),
                               comm="nccl", max_tokens=max_tokens)
        self.engine = self.trainer.engine
        self.engine.recompute = "full"
        first, last = self.pp_rank == 0, self.pp_rank == pp - 1
        self.first, self.last = first, last
        self.stage = PipelineStage(self._fwd, self.pp_rank, pp, None if first else rank - tp, None if last else rank + tp,
                                   device=self.dev, group=fwd, bwd_group=bwd, schedule=schedule,
                                   backward_fn=self._bwd, wgrad_fn=(lambda i: None))
        self.window = max(1, pp - self.pp_rank)
        self._states: Dict[int, object] = {}
        self._outs: List[dict] = []

    @staticmethod
    def _solo_group(world, rank):
        mine = None
        for r in range(world):
            g = dist.new_group([r])
            if r == rank:
                mine = g
        return mine

    # ---- the stage's computation per micro-batch ------------------------------------------------------------
    def _fwd(self, x_in, i):
        eng = self.engine
        st = eng.begin(self._batches[i], None, self._ce_norm, self._gen_norm, 1.0, True,
                       slot=f"mb{i % self.window}.", first=self.first, last=self.last)
        if self.first:
            eng.embed_fwd(st)
        else:
            st.xs[0] = x_in
        eng.layers_fwd(st)
        self._states[i] = st
        if self.last:
            out = eng.heads(st)
            self._outs.append(out)
            return out["loss"]
        return st.xs[-1]

    def _bwd(self, i, g):
        eng = self.engine
        st = self._states.pop(i)
        if not self.last:
            st.d_last = g
        eng.layers_bwd(st)
        if self.first:
            eng.embed_bwd(st)
            return None
        return st.d_first

    # ---- one optimizer step -----------------------------------------------------------------------------------
    def step(self, batches: Sequence[PackedBatch], lr: Optional[float] = None) -> Dict[str, torch.Tensor]:
        """``batches``: the micro-batches of this step, already on the device, the same on every rank.  Returns the
        summed losses on the last stage's ranks ({} elsewhere)."""
        self._batches = list(batches)
        self._ce_norm = max(sum(b.ce_weight_sum for b in batches), 1e-12)
        self._gen_norm = max(sum(b.gen_weight_sum for b in batches), 1.0)
        self.store.zero_grads()
        self._outs.clear()
        self.stage.run(len(batches))
        self.trainer.sync_tp_replicated_grads()
        self.trainer.optim.step(lr)
        out: Dict[str, torch.Tensor] = {}
        for o in self._outs:
            for k, v in o.items():
                out[k] = v if k not in out else out[k] + v
        return out
