#!/usr/bin/env python
"""Checkpoint conversion between the training layout and the Hugging Face layout.

    # training checkpoint (model_config.pt + model_wp{N}_pp0.pt [+ model_moe_layer*_expert*_wp0.pt], or the
    # model_tp{t}_pp{p}.pt files of a tensor x pipeline parallel run)  ->  HF directory
    python -m sensenova_u1_b200.train.convert to-hf --src RUN/job/1000 --tgt out/hf [--extras-from released/ckpt]

    # HF directory  ->  training shards for a weight-parallel size (and expert-parallel size for MoE models)
    python -m sensenova_u1_b200.train.convert to-train --src released/ckpt --tgt init/ckpt --wp 8 [--ep 8]
        [--mot-gen-init copy|keep]

Roles of the reference's ``tools/revert2hf.py:211-661`` (training -> HF: merge the weight-parallel shards, rename,
split fused tensors, 16-slice dense layout, one ``moemodel-*`` file per MoE layer, index) and of
``sensenovavl/utils/checkpoint.py:836-1407`` (HF -> shards, with the generation branch of a Mixture-of-Transformers
model initialised from the understanding branch when the source has none).  Both directions go through the flat
parameter store, so any shard count reads and any shard count writes."""
from __future__ import annotations

import argparse
import json
import re
import shutil
import sys
from pathlib import Path
from typing import List, Optional

import torch

_EXTRA_FILES = ("tokenizer.json", "tokenizer_config.json", "vocab.json", "merges.txt", "special_tokens_map.json",
                "added_tokens.json", "generation_config.json", "chat_template.json", "preprocessor_config.json")


def _config_from_training_dir(src: Path):
    from ..config import ModelConfig
    rec = torch.load(src / "model_config.pt", map_location="cpu", weights_only=False)
    mc = rec.get("model_config")
    if mc is None:
        raise ValueError(f"{src / 'model_config.pt'} was not written by this package (no 'model_config' entry); "
                         "convert reference checkpoints with the reference's own tool or load them through "
                         "CheckpointManager.load_model with a matching config")
    fields = {f for f in ModelConfig.__dataclass_fields__}
    return ModelConfig(**{k: v for k, v in mc.items() if k in fields})


def _load_tensor_pipeline_parts(srcp: Path, cfg, store, tp: int, pp: int) -> None:
    """Checkpoint of a tensor x pipeline parallel run: ``model_tp{t}_pp{p}.pt`` (``model_wp0_pp{p}.pt`` without tensor
    parallelism) hold stage ``p``'s layers under the model's own layer numbers, cut to rank ``t``'s heads and FFN units.
    Stages are merged over ``t``, their layers copied to their place; the front-ends and the token embedding come from
    the first stage, final norm and heads from the last (the stages that train them)."""
    from ..models.params import ParamStore
    from ..parallel.pipeline import partition_uniform
    from ..parallel.tensor_engine import merge_tp_stores, tp_local_config
    from . import ckpt_layout
    from .checkpoint import _shift_layers
    ranges = partition_uniform(cfg.num_layers, pp)
    for p_, (l0, l1) in enumerate(ranges):
        stage_cfg = cfg.replace(num_layers=l1 - l0)
        parts = []
        for t in range(tp):
            f = srcp / (f"model_tp{t}_pp{p_}.pt" if tp > 1 else f"model_wp0_pp{p_}.pt")
            if not f.exists():
                raise FileNotFoundError(f"{f}: the checkpoint is incomplete for tp {tp} x pp {pp}")
            part = ParamStore(tp_local_config(stage_cfg, tp), device="cpu", dtype=store.dtype, with_grads=False)
            ckpt_layout.load_train_state_dict(part, _shift_layers(torch.load(f, map_location="cpu", weights_only=False), -l0))
            parts.append(part)
        stage = merge_tp_stores(parts, stage_cfg) if tp > 1 else parts[0]
        for name, v in stage.p.items():
            if name.startswith("layers."):
                _, l, rest = name.split(".", 2)
                store.p[f"layers.{l0 + int(l)}.{rest}"].copy_(v)
            elif name.startswith(("final_norm", "lm_head", "fm_head", "mtp.")):
                if p_ == pp - 1:
                    store.p[name].copy_(v)
            elif p_ == 0:
                store.p[name].copy_(v)


def training_to_hf(src: str, tgt: str, extras_from: Optional[str] = None, max_shard_bytes: Optional[int] = None) -> List[str]:
    """Returns the names of the files written under ``tgt``."""
    from ..models.params import ParamStore
    from . import ckpt_layout
    from .checkpoint import export_hf
    srcp, tgtp = Path(src), Path(tgt)
    cfg = _config_from_training_dir(srcp)
    if cfg.is_moe and cfg.ep_size > 1:
        cfg = cfg.replace(ep_size=1)                      # the exported store holds every expert
    store = ParamStore(cfg, device="cpu", with_grads=False)
    names = [f.name for f in srcp.iterdir()]
    n_pp = 1 + max([int(m.group(1)) for n in names if (m := re.fullmatch(r"model_(?:wp|tp)\d+_pp(\d+)\.pt", n))] or [0])
    n_tp = 1 + max([int(m.group(1)) for n in names if (m := re.fullmatch(r"model_tp(\d+)_pp\d+\.pt", n))] or [-1])
    if n_pp > 1 or n_tp > 0:
        _load_tensor_pipeline_parts(srcp, cfg, store, max(n_tp, 1), n_pp)
    else:
        pat = re.compile(r"model_(wp|tp)(\d+)_pp0\.pt")
        files = sorted((int(m.group(2)), f) for f in srcp.iterdir() if (m := pat.fullmatch(f.name)))
        if not files:
            raise FileNotFoundError(f"no model_wp*_pp0.pt / model_tp*_pp0.pt in {srcp}")
        shards = [torch.load(f, map_location="cpu", weights_only=False) for _, f in files]
        ckpt_layout.load_train_state_dict(store, ckpt_layout.merge_shards(shards))
    if cfg.is_moe:
        epat = re.compile(r"model_moe_layer(\d+)_expert(\d+)_wp0\.pt")
        by_layer = {}
        for f in srcp.iterdir():
            m = epat.fullmatch(f.name)
            if m:
                by_layer.setdefault(int(m.group(1)), []).append((int(m.group(2)), f))
        if len(by_layer) != 2 * cfg.num_layers:
            raise FileNotFoundError(f"{srcp}: expert files of {len(by_layer)} of {2 * cfg.num_layers} MoE layers found")
        for lid, lst in sorted(by_layer.items()):
            parts = [torch.load(f, map_location="cpu", weights_only=False) for _, f in sorted(lst)]
            merged = {k: torch.cat([p[k] for p in parts], dim=0) for k in parts[0]}     # expert-parallel ranks in order
            ckpt_layout.load_expert_file(store, lid // 2, bool(lid % 2), merged)
    tgtp.mkdir(parents=True, exist_ok=True)
    export_hf(store, str(tgtp), max_shard_bytes=max_shard_bytes)
    if extras_from:
        for name in _EXTRA_FILES:
            f = Path(extras_from) / name
            if f.is_file():
                shutil.copy2(f, tgtp / name)
    return sorted(p.name for p in tgtp.iterdir())


def hf_to_training(src: str, tgt: str, wp: int = 1, ep: int = 1, mot_gen_init: str = "keep") -> List[str]:
    """HF directory -> ``model_wp{r}_pp0.pt`` for r < wp, expert files per expert-parallel rank, ``model_config.pt``.
    ``mot_gen_init="copy"`` overwrites the generation branch of the decoder with the understanding branch (the
    reference's initialisation of a Mixture-of-Transformers model from an understanding-only checkpoint,
    ``mot_random_init=False``)."""
    from ..models.params import GEN, UND
    from . import ckpt_layout
    from .checkpoint import import_hf
    store = import_hf(src, device="cpu", with_grads=False, strict=mot_gen_init != "copy")
    cfg = store.cfg
    if mot_gen_init == "copy":
        for name, t in store.p.items():
            if ".moe_gen." in name:                       # mixtures of equal shape only; a smaller one keeps its init
                u = store.p[name.replace(".moe_gen.", ".moe_und.")]
                if u.shape == t.shape:
                    t.copy_(u)
            elif ".moe_und." not in name and name.startswith(("layers.", "final_norm")) and t.dim() > 1 and t.shape[0] == 2:
                t[GEN].copy_(t[UND])
    elif mot_gen_init != "keep":
        raise ValueError("mot_gen_init is 'keep' or 'copy'")
    tgtp = Path(tgt)
    tgtp.mkdir(parents=True, exist_ok=True)
    full = ckpt_layout.train_state_dict(store)
    for r in range(wp):
        torch.save({k: v.clone() for k, v in ckpt_layout.shard_state_dict(full, r, wp).items()}, tgtp / f"model_wp{r}_pp0.pt")
        (tgtp / f"topo_wp{r}_pp0.json").write_text(json.dumps({"tp": 0, "pp": 0, "wp": r, "wp_size": wp, "model": cfg.name}))
    if cfg.is_moe:
        if ep < 1 or cfg.num_experts % ep or cfg.gen_num_experts % ep:
            raise ValueError(f"expert counts {cfg.num_experts} / {cfg.gen_num_experts} do not split over {ep} ranks")
        for name, sd in ckpt_layout.expert_files(store):          # one file per (layer, branch) holding every expert
            m = re.fullmatch(r"model_moe_layer(\d+)_expert0_wp0\.pt", name)
            for e in range(ep):
                part = {k: v.chunk(ep, dim=0)[e].clone() for k, v in sd.items()}
                torch.save(part, tgtp / f"model_moe_layer{m.group(1)}_expert{e}_wp0.pt")
    torch.save(ckpt_layout.model_config_record(cfg if ep == 1 else cfg.replace(ep_size=ep)), tgtp / "model_config.pt")
    return sorted(p.name for p in tgtp.iterdir())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0], formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("to-hf", help="training checkpoint -> Hugging Face directory")
    a.add_argument("--src", required=True)
    a.add_argument("--tgt", required=True)
    a.add_argument("--extras-from", default=None, help="HF directory to copy tokenizer / generation config files from")
    a.add_argument("--max-shard-gb", type=float, default=None)
    b = sub.add_parser("to-train", help="Hugging Face directory -> training shards")
    b.add_argument("--src", required=True)
    b.add_argument("--tgt", required=True)
    b.add_argument("--wp", type=int, default=1, help="weight-parallel size of the shards")
    b.add_argument("--ep", type=int, default=1, help="expert-parallel size (MoE models)")
    b.add_argument("--mot-gen-init", default="keep", choices=["keep", "copy"])
    args = ap.parse_args(argv)
    if args.cmd == "to-hf":
        names = training_to_hf(args.src, args.tgt, args.extras_from,
                               int(args.max_shard_gb * (1 << 30)) if args.max_shard_gb else None)
    else:
        names = hf_to_training(args.src, args.tgt, args.wp, args.ep, args.mot_gen_init)
    print(f"wrote {len(names)} files to {args.tgt}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
