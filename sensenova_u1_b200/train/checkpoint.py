"""Checkpoints: training snapshots (per-rank shards + markers, resumable) and HF safetensors
import / export.

Training directory layout follows the reference (training/sensenovalm/checkpoint/components.py:
111-832, checkpoint_manager.py:441-786): ``{folder}/{step}/`` or ``{folder}/snapshot/{0,1}/`` with

    model_tp{t}_pp{p}.pt / model_wp{w}_pp{p}.pt   weights (flat arenas; written by data-parallel rank 0)
    topo_*.json                                   shard topology
    optimizer_*_zo{z}.pt                          this rank's ZeRO partition (state + remainders)
    averaged_model/...                            EMA shadow of the local partition
    context.pt, schedulder.pt [sic], sampler.pt   train state, LR schedule, data state
    {step}.step                                   written last: marks the checkpoint complete

HF layout (src/sensenova_u1 loader, training/tools/revert2hf.py:347-405): safetensors shards +
``model.safetensors.index.json`` + ``config.json`` with the per-module key names of
``models/params.py::hf_state_dict``.
"""
from __future__ import annotations

import json
import os
import re
import signal
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..config import ModelConfig
from ..models.params import ParamStore, hf_state_dict, load_hf_state_dict


def _is_dist():
    return dist.is_available() and dist.is_initialized()


def _rank():
    return dist.get_rank() if _is_dist() else 0


def _atomic_save(obj, path: Path):
    tmp = path.with_suffix(path.suffix + ".tmp")
    torch.save(obj, tmp)
    os.replace(tmp, path)


@dataclass
class LoadMask:
    """What to restore from a checkpoint (reference: CheckpointLoadMask, checkpoint_manager.py:200-249)."""
    model: bool = True
    optimizer: bool = False
    sampler: bool = False
    scheduler: bool = False

    @classmethod
    def parse(cls, content) -> "LoadMask":
        items = {content} if isinstance(content, str) else set(content)
        if "all" in items:
            return cls(True, True, True, True)
        bad = items - {"model", "optimizer", "sampler", "scheduler"}
        if bad:
            raise ValueError(f"unknown load_ckpt_info.content entries: {sorted(bad)}")
        return cls("model" in items, "optimizer" in items, "sampler" in items, "scheduler" in items)


class CheckpointManager:
    def __init__(self, folder: str, checkpoint_every: int = 0, snapshot_every: int = 0,
                 stop_file_path: Optional[str] = None, auto_resume: bool = True, tp_rank=0, pp_rank=0,
                 wp_rank: Optional[int] = None, dp_rank=0, zero_rank=0):
        self.folder = Path(folder.split(":", 1)[1] if folder.startswith("local:") else folder)
        self.every, self.snap_every = checkpoint_every, snapshot_every
        self.stop_file = Path(stop_file_path) if stop_file_path else None
        self.auto_resume = auto_resume
        self.tp, self.pp, self.wp, self.dp, self.zo = tp_rank, pp_rank, wp_rank, dp_rank, zero_rank
        self.snap_idx = 0
        self._quit = False
        try:
            signal.signal(signal.SIGUSR1, lambda *_: setattr(self, "_quit", True))
        except ValueError:
            pass  # not in the main thread

    # ---- policy --------------------------------------------------------------
    def decide(self, step: int, total_steps: int):
        """Returns (save?, kind, stop?).  A stop file / SIGUSR1 seen by any rank stops all of them."""
        stop = self._quit or (self.stop_file is not None and self.stop_file.exists())
        if _is_dist():
            t = torch.tensor([1 if stop else 0])
            if dist.get_backend() == "nccl":
                t = t.cuda()
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            stop = bool(t.item())
        if stop or step == total_steps:
            return True, "step", stop
        if self.every and step % self.every == 0:
            return True, "step", False
        if self.snap_every and step % self.snap_every == 0:
            return True, "snapshot", False
        return False, "", False

    def _dir(self, step: int, kind: str) -> Path:
        if kind == "snapshot":
            d = self.folder / "snapshot" / str(self.snap_idx)
            self.snap_idx = 1 - self.snap_idx
            return d
        return self.folder / str(step)

    def _model_name(self):
        return f"model_wp{self.wp}_pp{self.pp}.pt" if self.wp is not None else f"model_tp{self.tp}_pp{self.pp}.pt"

    def _optim_name(self):
        a = f"wp{self.wp}" if self.wp is not None else f"tp{self.tp}"
        return f"optimizer_{a}_pp{self.pp}_zo{self.zo}.pt"

    # ---- save ------------------------------------------------------------------
    def save(self, step: int, store: ParamStore, optim=None, train_state: Optional[dict] = None,
             scheduler_state: Optional[dict] = None, sampler_state: Optional[dict] = None, ema=None,
             kind: str = "step") -> Path:
        d = self._dir(step, kind)
        d.mkdir(parents=True, exist_ok=True)
        for old in d.glob("*.step"):
            old.unlink()
        if self.dp == 0:
            _atomic_save({k: v.detach().cpu() for k, v in store.arena.items()}, d / self._model_name())
            topo = {"tp": self.tp, "pp": self.pp, "wp": self.wp, "sizes": store.sizes,
                    "model": store.cfg.name, "offsets": {k: list(v) for k, v in store.offsets.items()}}
            (d / self._model_name().replace("model_", "topo_").replace(".pt", ".json")).write_text(json.dumps(topo))
        if optim is not None:
            _atomic_save(optim.state_dict(), d / self._optim_name())
        if ema is not None:
            (d / "averaged_model").mkdir(exist_ok=True)
            _atomic_save({k: v.cpu() for k, v in ema.items()}, d / "averaged_model" / self._optim_name().replace("optimizer_", "model_"))
            if _rank() == 0:
                (d / "averaged_model" / "averaged_model_info.json").write_text(json.dumps({"step": step}))
        if sampler_state is not None:
            _atomic_save(sampler_state, d / (f"sampler_{self.dp}.pt"))
        if _rank() == 0:
            if train_state is not None:
                _atomic_save(train_state, d / "context.pt")
            if scheduler_state is not None:
                _atomic_save(scheduler_state, d / "schedulder.pt")
            _atomic_save({"model_config": store.cfg.__dict__}, d / "model_config.pt")
        if _is_dist():
            dist.barrier()
        if _rank() == 0:
            (d / f"{step}.step").write_text(str(time.time()))
        if _is_dist():
            dist.barrier()
        return d

    # ---- resume -----------------------------------------------------------------
    def latest(self) -> Optional[Path]:
        """Newest complete checkpoint (a directory that holds a ``*.step`` marker)."""
        best, best_step = None, -1
        if not self.folder.exists():
            return None
        for marker in self.folder.glob("**/*.step"):
            m = re.fullmatch(r"(\d+)\.step", marker.name)
            if m and int(m.group(1)) > best_step:
                best, best_step = marker.parent, int(m.group(1))
        return best

    def load(self, d: Path, store: ParamStore, optim=None, mask: LoadMask = LoadMask()):
        """Restores the parts selected by ``mask``; returns (train_state, scheduler_state, sampler_state)."""
        out = [None, None, None]
        if mask.model:
            sd = torch.load(d / self._model_name(), map_location="cpu")
            for k, v in sd.items():
                if store.arena[k].numel() != v.numel():
                    raise ValueError(f"arena {k}: checkpoint has {v.numel()} elements, model {store.arena[k].numel()}")
                store.arena[k].copy_(v)
        if mask.optimizer and optim is not None:
            optim.load_state_dict(torch.load(d / self._optim_name(), map_location="cpu"))
        if (d / "context.pt").exists():
            out[0] = torch.load(d / "context.pt", map_location="cpu")
        if mask.scheduler and (d / "schedulder.pt").exists():
            out[1] = torch.load(d / "schedulder.pt", map_location="cpu")
        if mask.sampler and (d / f"sampler_{self.dp}.pt").exists():
            out[2] = torch.load(d / f"sampler_{self.dp}.pt", map_location="cpu")
        return tuple(out)

    def try_resume(self, store, optim=None, mask: Optional[LoadMask] = None):
        if not self.auto_resume:
            return None
        d = self.latest()
        if d is None:
            return None
        return d, self.load(d, store, optim, mask or LoadMask(True, True, True, True))


# ---------------------------------------------------------------------------
# HF safetensors
# ---------------------------------------------------------------------------
def hf_config_dict(cfg: ModelConfig) -> dict:
    llm = {"hidden_size": cfg.hidden_size, "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads,
           "head_dim": cfg.head_dim, "intermediate_size": cfg.ffn_size, "num_hidden_layers": cfg.num_layers,
           "vocab_size": cfg.vocab_size, "rms_norm_eps": cfg.rms_eps, "rope_theta": cfg.rope_base,
           "rope_theta_hw": cfg.rope_base_hw, "max_position_embeddings": cfg.max_position_embeddings}
    if cfg.is_moe:
        llm.update(num_experts=cfg.num_experts, num_experts_per_tok=cfg.num_experts_per_tok,
                   gen_num_experts=cfg.gen_num_experts, gen_num_experts_per_tok=cfg.gen_num_experts_per_tok,
                   moe_intermediate_size=cfg.moe_intermediate_size, gen_moe_intermediate_size=cfg.moe_intermediate_size,
                   norm_topk_prob=cfg.norm_topk_prob)
    return {"model_type": "neo_chat", "architectures": ["NEOChatModel"], "llm_config": llm,
            "vision_config": {"patch_size": cfg.patch_size, "hidden_size": cfg.vision_hidden,
                              "downsample_ratio": 1.0 / cfg.merge_size, "rope_theta_vision": cfg.rope_theta_vision,
                              "llm_hidden_size": cfg.hidden_size, "num_hidden_layers": 0},
            "downsample_ratio": 1.0 / cfg.merge_size, "noise_scale": cfg.noise_scale,
            "noise_scale_mode": cfg.noise_scale_mode, "noise_scale_base_image_seq_len": cfg.noise_scale_base_image_seq_len,
            "noise_scale_max_value": cfg.noise_scale_max_value, "add_noise_scale_embedding": cfg.add_noise_scale_embedding,
            "t_eps": cfg.t_eps, "time_schedule": cfg.time_schedule, "time_shift_type": cfg.time_shift_type,
            "base_shift": cfg.base_shift, "max_shift": cfg.max_shift, "base_image_seq_len": cfg.base_image_seq_len,
            "max_image_seq_len": cfg.max_image_seq_len, "use_pixel_head": False, "sensenova_u1_min_version": "0.1.0",
            "fm_head_dim": cfg.fm_head_dim, "timestep_freq_dim": cfg.timestep_freq_dim}


def config_from_hf(d: dict, **overrides) -> ModelConfig:
    llm, vis = d["llm_config"], d.get("vision_config", {})
    kw = dict(name=d.get("_name_or_path", "hf-checkpoint"), hidden_size=llm["hidden_size"], num_heads=llm["num_attention_heads"],
              num_kv_heads=llm["num_key_value_heads"], head_dim=llm.get("head_dim", llm["hidden_size"] // llm["num_attention_heads"]),
              ffn_size=llm["intermediate_size"], num_layers=llm["num_hidden_layers"], vocab_size=llm["vocab_size"],
              rms_eps=llm.get("rms_norm_eps", 1e-6), rope_base=llm.get("rope_theta", 5e6), rope_base_hw=llm.get("rope_theta_hw", 1e4),
              patch_size=vis.get("patch_size", 16), vision_hidden=vis.get("hidden_size", 1024),
              merge_size=int(round(1 / d.get("downsample_ratio", 0.5))),
              num_experts=llm.get("num_experts", 0) or 0, num_experts_per_tok=llm.get("num_experts_per_tok", 0) or 0,
              gen_num_experts=llm.get("gen_num_experts", 0) or 0, gen_num_experts_per_tok=llm.get("gen_num_experts_per_tok", 0) or 0,
              moe_intermediate_size=llm.get("moe_intermediate_size", 0) or 0)
    for k in ("noise_scale", "noise_scale_mode", "noise_scale_base_image_seq_len", "noise_scale_max_value",
              "add_noise_scale_embedding", "t_eps", "time_schedule", "time_shift_type", "base_shift", "max_shift",
              "base_image_seq_len", "max_image_seq_len", "fm_head_dim", "timestep_freq_dim"):
        if k in d:
            kw[k] = d[k]
    kw.update(overrides)
    return ModelConfig(**kw)


def export_hf(store: ParamStore, out_dir: str, max_shard_bytes: int = 4 << 30) -> Dict[str, str]:
    """Writes ``model-XXXXX-of-YYYYY.safetensors`` + index + config.json; returns the weight map."""
    from safetensors.torch import save_file
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    sd = hf_state_dict(store)
    shards, cur, cur_bytes = [], {}, 0
    for k, v in sd.items():
        nb = v.numel() * v.element_size()
        if cur and cur_bytes + nb > max_shard_bytes:
            shards.append(cur); cur, cur_bytes = {}, 0
        cur[k] = v.detach().to("cpu").contiguous()
        cur_bytes += nb
    if cur:
        shards.append(cur)
    weight_map = {}
    for i, sh in enumerate(shards):
        name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, str(out / name), metadata={"format": "pt"})
        weight_map.update({k: name for k in sh})
    total = sum(v.numel() * v.element_size() for v in sd.values())
    (out / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}, indent=1))
    (out / "config.json").write_text(json.dumps(hf_config_dict(store.cfg), indent=1))
    return weight_map


def import_hf(model_dir: str, device="cpu", dtype=torch.bfloat16, with_grads=False, strict=True, **cfg_overrides) -> ParamStore:
    """Builds a ParamStore from an HF checkpoint directory (safetensors shards + config.json)."""
    from safetensors import safe_open
    d = Path(model_dir)
    cfg = config_from_hf(json.loads((d / "config.json").read_text()), **cfg_overrides)
    store = ParamStore(cfg, device=device, dtype=dtype, with_grads=with_grads)
    files = sorted(d.glob("*.safetensors"))
    sd = {}
    for f in files:
        with safe_open(str(f), framework="pt", device="cpu") as fh:
            for k in fh.keys():
                sd[k] = fh.get_tensor(k)
    load_hf_state_dict(store, sd, strict=strict)
    return store
