"""Checkpoints: training snapshots (per-rank shards + markers, resumable) and HF safetensors
import / export.

Training directory layout follows the reference (training/sensenovalm/checkpoint/components.py:
111-832, checkpoint_manager.py:441-786): ``{folder}/{step}/`` or ``{folder}/snapshot/{0,1}/`` with

    model_wp{w}_pp{p}.pt (model_tp{t}_pp{p}.pt)    weights: a state dict in the reference's training key
                                                  names, rows split over the weight-parallel group
                                                  (train/ckpt_layout.py); written by data-parallel rank 0
    model_moe_layer{2l+gen}_expert{e}_wp{w}.pt    the experts of expert-parallel rank e, one file per MoE module
    model_config.pt, topo_*.json                  model configuration, shard topology
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
from . import ckpt_layout


def _is_dist():
    return dist.is_available() and dist.is_initialized()


def _rank():
    return dist.get_rank() if _is_dist() else 0


def _atomic_save(obj, path: Path):
    tmp = path.with_suffix(path.suffix + ".tmp")
    torch.save(obj, tmp)
    os.replace(tmp, path)


class RemoteMirror:
    """Copies checkpoint directories to a storage back-end (``utils/storage.py``: ``s3:bucket/prefix`` or any scheme
    registered there) on a background thread, and fetches the newest complete one for a resume.  The job itself always
    writes to, and reads from, a local working folder; the training loop pays for the serialisation only (the
    reference stages through ``/dev/shm`` and uploads asynchronously: utils/storage_manager.py:105-1281,
    ``ckpt.async_upload``).  A directory counts as complete remotely once its ``<step>.step`` marker is there; the
    marker is sent after every rank has confirmed its own uploads (at the next save, or at ``close``)."""

    def __init__(self, url: str, local_root: Path):
        import queue
        import threading
        from ..utils.storage import split_url
        self.backend, self.base = split_url(url)
        self.base = self.base.rstrip("/")
        self.local_root = Path(local_root)
        self.q: "queue.Queue" = queue.Queue()
        self.errors = []
        self.pending_marker: Optional[Path] = None
        self.t = threading.Thread(target=self._loop, daemon=True)
        self.t.start()

    def _remote(self, f: Path) -> str:
        return self.base + "/" + f.relative_to(self.local_root).as_posix()

    def _loop(self):
        while True:
            f = self.q.get()
            if f is None:
                return
            try:
                self.backend.upload(str(f), self._remote(f))
            except Exception as e:                    # reported by confirm(); the thread keeps serving
                self.errors.append(f"{f.name}: {type(e).__name__}: {e}")
            finally:
                self.q.task_done()

    def push(self, files) -> None:
        for f in files:
            self.q.put(Path(f))

    def confirm(self) -> None:
        """Waits for this rank's uploads, then (all ranks together) lets rank 0 send the marker of the last save."""
        self.q.join()
        failed = bool(self.errors)
        if _is_dist():
            t = torch.tensor([1 if failed else 0])
            if dist.get_backend() == "nccl":
                t = t.cuda()
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            failed = bool(t.item())
        if self.pending_marker is not None and not failed and _rank() == 0:
            self.backend.upload(str(self.pending_marker), self._remote(self.pending_marker))
        self.pending_marker = None
        if self.errors:
            errs, self.errors = self.errors, []
            raise IOError("checkpoint upload failed (the remote copy has no marker and will be ignored): " + "; ".join(errs))

    def close(self) -> None:
        try:
            self.confirm()
        finally:
            self.q.put(None)
            self.t.join(timeout=5)

    def pull_latest(self) -> Optional[Path]:
        """Downloads the newest remote directory that has a marker into the local folder; returns its local path."""
        best, best_step = None, -1
        tops = self.backend.listdir(self.base)
        cands = [(n,) for n in tops if n.isdigit()] + [("snapshot", n) for n in (self.backend.listdir(self.base + "/snapshot")
                                                                               if "snapshot" in tops else [])]
        for parts in cands:
            rel = "/".join(parts)
            for name in self.backend.listdir(self.base + "/" + rel):
                m = re.fullmatch(r"(\d+)\.step", name)
                if m and int(m.group(1)) > best_step:
                    best, best_step = rel, int(m.group(1))
        if best is None:
            return None
        dst = self.local_root / best
        if _rank() == 0:
            self._fetch(self.base + "/" + best, dst)
        if _is_dist():
            dist.barrier()
        return dst

    def _fetch(self, remote_dir: str, dst: Path) -> None:
        dst.mkdir(parents=True, exist_ok=True)
        names = self.backend.listdir(remote_dir)
        for name in sorted(names, key=lambda n: n.endswith(".step")):       # the marker last, as when it was written
            r = remote_dir + "/" + name
            if self.backend.listdir(r):                                      # a sub-directory (averaged_model/)
                self._fetch(r, dst / name)
            else:
                self.backend.download(r, str(dst / name))


_LAYER_KEY = re.compile(r"(\blayers\.)(\d+)(\.)")


def _shift_layers(sd: dict, offset: int) -> dict:
    """Adds ``offset`` to the decoder-layer index in every key (a pipeline stage numbers its layers from 0)."""
    if not offset:
        return sd
    return {_LAYER_KEY.sub(lambda m: f"{m.group(1)}{int(m.group(2)) + offset}{m.group(3)}", k, count=1): v for k, v in sd.items()}


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
                 wp_rank: Optional[int] = None, dp_rank=0, zero_rank=0, wp_size: int = 1, tp_size: int = 1,
                 ep_rank: int = 0, expert_dp_rank: int = 0, layer_offset: int = 0, local_work_folder: Optional[str] = None):
        """``folder``: ``local:path`` / a plain path, or a remote URL of a registered storage back-end (``s3:bucket/run``):
        then checkpoints are written under ``local_work_folder`` (``ckpt.async_upload_tmp_folder``) and mirrored.
        ``layer_offset``: index of this pipeline stage's first decoder layer (a stage numbers its layers from 0;
        the files carry the model's numbering).  ``wp_rank / wp_size``: position in the weight-parallel group (None / 1: weights are whole on every rank and
        data-parallel rank 0 writes them as the single shard ``model_wp0``); ``ep_rank``: which experts this rank holds,
        ``expert_dp_rank``: 0 on exactly one rank per expert-parallel rank (that one writes the expert files)."""
        self.mirror: Optional[RemoteMirror] = None
        scheme = folder.split(":", 1)[0] if ":" in folder else "local"
        if scheme not in ("local", "file") and len(scheme) > 1 and not os.path.exists(folder):
            # a remote destination: work in a local folder, mirror every save to the remote on a background thread
            work = Path(local_work_folder or os.path.join("RUN", "_ckpt_work", re.sub(r"[^A-Za-z0-9_.-]+", "_", folder)))
            self.mirror = RemoteMirror(folder, work)
            folder = str(work)
        self.folder = Path(folder.split(":", 1)[1] if folder.startswith(("local:", "file:")) else folder)
        self.every, self.snap_every = checkpoint_every, snapshot_every
        self.stop_file = Path(stop_file_path) if stop_file_path else None
        self.auto_resume = auto_resume
        self.tp, self.pp, self.wp, self.dp, self.zo = tp_rank, pp_rank, wp_rank, dp_rank, zero_rank
        self.wp_size, self.tp_size, self.ep, self.edp = wp_size, tp_size, ep_rank, expert_dp_rank
        self.layer_offset = int(layer_offset)
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
        if self.tp_size > 1:
            return f"model_tp{self.tp}_pp{self.pp}.pt"
        return f"model_wp{self.wp or 0}_pp{self.pp}.pt"

    def _optim_name(self):
        a = f"tp{self.tp}" if self.tp_size > 1 else f"wp{self.wp or 0}"
        return f"optimizer_{a}_pp{self.pp}_zo{self.zo}.pt"

    # ---- save ------------------------------------------------------------------
    def save(self, step: int, store: ParamStore, optim=None, train_state: Optional[dict] = None,
             scheduler_state: Optional[dict] = None, sampler_state: Optional[dict] = None, ema=None,
             kind: str = "step", model_cfg: Optional[ModelConfig] = None) -> Path:
        """``model_cfg``: the whole model's configuration when ``store`` holds a part of it (a pipeline stage, a
        tensor-parallel slice); it is what ``model_config.pt`` records."""
        if self.mirror is not None:
            self.mirror.confirm()                 # the previous save's uploads are done everywhere: its marker goes out
        d = self._dir(step, kind)
        d.mkdir(parents=True, exist_ok=True)
        written = []                              # files of this rank, for the mirror

        def put(obj, path: Path):
            _atomic_save(obj, path)
            written.append(path)

        def put_text(text: str, path: Path):
            path.write_text(text)
            written.append(path)
        # a reused snapshot directory: the old marker goes first (one rank), then everybody may write
        if _rank() == 0:
            for old in d.glob("*.step"):
                old.unlink(missing_ok=True)
        if _is_dist():
            dist.barrier()
        if hasattr(store, "to_param_store"):
            store = store.to_param_store()       # weight parallel: assemble the full tensors (collective), slice below
        if self.dp == 0:
            full = ckpt_layout.train_state_dict(store)
            shard = ckpt_layout.shard_state_dict(full, self.wp or 0, self.wp_size if self.wp is not None else 1)
            shard = _shift_layers(shard, self.layer_offset)
            put({k: v.cpu() for k, v in shard.items()}, d / self._model_name())
            topo = {"tp": self.tp, "pp": self.pp, "wp": self.wp, "wp_size": self.wp_size, "model": store.cfg.name,
                    "layout": "state dict, training key names; rows split over wp"}
            put_text(json.dumps(topo), d / self._model_name().replace("model_", "topo_").replace(".pt", ".json"))
        if store.cfg.is_moe and self.edp == 0 and (store.cfg.ep_size > 1 or self.dp == 0):
            for name, sd in ckpt_layout.expert_files(store):
                put({k: v.cpu() for k, v in sd.items()}, d / name)
        if optim is not None:
            put(optim.state_dict(), d / self._optim_name())
        if ema is not None:
            (d / "averaged_model").mkdir(exist_ok=True)
            put({k: v.cpu() for k, v in ema.items()}, d / "averaged_model" / self._optim_name().replace("optimizer_", "model_"))
            if _rank() == 0:
                put_text(json.dumps({"step": step}), d / "averaged_model" / "averaged_model_info.json")
        if sampler_state is not None:
            put(sampler_state, d / (f"sampler_{self.dp}.pt"))
        if _rank() == 0:
            if train_state is not None:
                put(train_state, d / "context.pt")
            if scheduler_state is not None:
                put(scheduler_state, d / "schedulder.pt")
            put(ckpt_layout.model_config_record(model_cfg or store.cfg), d / "model_config.pt")
        if _is_dist():
            dist.barrier()
        if _rank() == 0:
            (d / f"{step}.step").write_text(str(time.time()))
        if _is_dist():
            dist.barrier()
        if self.mirror is not None:
            self.mirror.push(written)
            self.mirror.pending_marker = d / f"{step}.step"
        return d

    def ping(self) -> None:
        """Fails now, not at the first save, when the checkpoint folder (and the remote destination) cannot be written
        (the reference's storage "ping" at start-up, checkpoint_manager.py:795)."""
        self.folder.mkdir(parents=True, exist_ok=True)
        f = self.folder / f".ping_{_rank()}"
        f.write_text(str(time.time()))
        try:
            if self.mirror is not None:
                self.mirror.backend.upload(str(f), self.mirror._remote(f))
        finally:
            f.unlink(missing_ok=True)

    def close(self) -> None:
        """Finishes outstanding uploads (a remote destination only)."""
        if self.mirror is not None:
            self.mirror.close()

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
            self.load_model(d, store)
        if mask.optimizer and optim is not None:
            optim.load_state_dict(torch.load(d / self._optim_name(), map_location="cpu"))
        if (d / "context.pt").exists():
            out[0] = torch.load(d / "context.pt", map_location="cpu")
        if mask.scheduler and (d / "schedulder.pt").exists():
            out[1] = torch.load(d / "schedulder.pt", map_location="cpu")
        if mask.sampler and (d / f"sampler_{self.dp}.pt").exists():
            out[2] = torch.load(d / f"sampler_{self.dp}.pt", map_location="cpu")
        return tuple(out)

    def load_ema(self, d: Path) -> Optional[Dict[str, torch.Tensor]]:
        """This rank's EMA shadow of checkpoint ``d`` (None when the checkpoint has none for this rank; the reference
        restores its averaged model from the same folder, core/model_average.py:251-273)."""
        f = Path(d) / "averaged_model" / self._optim_name().replace("optimizer_", "model_")
        return torch.load(f, map_location="cpu", weights_only=False) if f.exists() else None

    def load_model(self, d: Path, store: ParamStore) -> None:
        """Reads every weight-parallel shard that the directory holds (whatever their number: a checkpoint
        written at one parallel layout loads at another, also one written by the reference), merges them and fills
        the arenas; then this rank's experts."""
        if hasattr(store, "load_from"):
            # weight parallel: read into a full store first, then keep this rank's pieces
            full = ParamStore(store.cfg, device=store.device, dtype=store.dtype, with_grads=False)
            self.load_model(d, full)
            store.load_from(full)
            return
        if self.tp_size > 1:
            # tensor parallel: the file holds this rank's column / row slices as they are; nothing to merge
            f = d / self._model_name()
            if not f.exists():
                raise FileNotFoundError(f"{f}: the checkpoint was written at another tensor / pipeline layout")
            shards = [torch.load(f, map_location="cpu", weights_only=False)]
        else:
            pat = re.compile(r"model_(wp|tp)(\d+)_pp%d\.pt" % self.pp)
            files = sorted((int(m.group(2)), f) for f in d.iterdir() if (m := pat.fullmatch(f.name)))
            if not files:
                raise FileNotFoundError(f"no model_wp*_pp{self.pp}.pt / model_tp*_pp{self.pp}.pt in {d}")
            shards = [torch.load(f, map_location="cpu", weights_only=False) for _, f in files]
        ckpt_layout.load_train_state_dict(store, _shift_layers(ckpt_layout.merge_shards(shards), -self.layer_offset))
        cfg = store.cfg
        if cfg.is_moe:
            ep = store.ep_rank if cfg.ep_size > 1 else 0
            for l in range(cfg.num_layers):
                for gen in (False, True):
                    f = d / ckpt_layout.expert_file_name(l, gen, ep)
                    if not f.exists():
                        raise FileNotFoundError(f"{f}: the checkpoint has no experts for expert-parallel rank {ep} "
                                                f"(it was written with another expert-parallel size)")
                    ckpt_layout.load_expert_file(store, l, gen, torch.load(f, map_location="cpu", weights_only=False))

    def try_resume(self, store, optim=None, mask: Optional[LoadMask] = None):
        if not self.auto_resume:
            return None
        d = self.latest()
        if d is None and self.mirror is not None:
            d = self.mirror.pull_latest()          # a fresh machine: fetch the newest complete remote checkpoint
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
              num_experts=llm.get("num_experts", llm.get("num_local_experts", 0)) or 0, num_experts_per_tok=llm.get("num_experts_per_tok", 0) or 0,
              gen_num_experts=llm.get("gen_num_experts", 0) or 0, gen_num_experts_per_tok=llm.get("gen_num_experts_per_tok", 0) or 0,
              moe_intermediate_size=llm.get("moe_intermediate_size", 0) or 0)
    for k in ("noise_scale", "noise_scale_mode", "noise_scale_base_image_seq_len", "noise_scale_max_value",
              "add_noise_scale_embedding", "t_eps", "time_schedule", "time_shift_type", "base_shift", "max_shift",
              "base_image_seq_len", "max_image_seq_len", "fm_head_dim", "timestep_freq_dim"):
        if k in d:
            kw[k] = d[k]
    kw.update(overrides)
    return ModelConfig(**kw)


def _dense_slice_of(key: str, num_layers: int) -> int:
    """Slice number (1-based, of 16 or 17) of a non-expert tensor in the layout of the released checkpoints, which
    the reference's converter writes (training/tools/revert2hf.py:347-405): three vision-encoder slices (empty: the
    encoder has no layers; the patch embeddings sit in the first), one connector slice (empty), one for the
    flow-matching modules, then the decoder in ten slices of ``num_layers // 10`` layers plus one for the rest;
    embedding, final norms and head travel with the first decoder slice."""
    if key.startswith("vision_model"):
        return 1
    if key.startswith("fm_modules"):
        return 5
    m = re.search(r"\.layers\.(\d+)\.", key)
    if m is None:
        return 6
    per = max(1, num_layers // 10)
    return 6 + min(int(m.group(1)) // per, 10)


def export_hf(store: ParamStore, out_dir: str, max_shard_bytes: Optional[int] = None, group=None) -> Dict[str, str]:
    """Writes the HF checkpoint: safetensors shards + ``model.safetensors.index.json`` + ``config.json``; returns the
    weight map (rank 0; other ranks return their own part).

    Default layout = the released checkpoints' (see :func:`_dense_slice_of`): ``model-000NN-of-000MM.safetensors`` for
    everything but the experts and ``moemodel-*.safetensors`` for the experts, one file per MoE layer.  With expert
    parallelism every expert-parallel rank writes the experts it holds to ``moemodel-ep{r}-of-{n}.safetensors`` and
    rank 0 merges all ranks' entries into the index, so the checkpoint is complete whatever the layout of the job
    (call it on every rank of ``group``).  ``max_shard_bytes`` switches the non-expert part to plain size-bounded
    shards."""
    from safetensors.torch import save_file
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    cfg = store.cfg
    sd = hf_state_dict(store)
    dense = {k: v for k, v in sd.items() if ".experts." not in k}
    experts = {k: v for k, v in sd.items() if ".experts." in k}
    ep = cfg.ep_size if (cfg.is_moe and cfg.ep_size > 1) else 1
    rank = _rank()
    weight_map: Dict[str, str] = {}

    def cpu(v):
        return v.detach().to("cpu").contiguous()
    if rank == 0:
        if max_shard_bytes:
            shards, cur, cur_bytes = [], {}, 0
            for k, v in dense.items():
                nb = v.numel() * v.element_size()
                if cur and cur_bytes + nb > max_shard_bytes:
                    shards.append(cur); cur, cur_bytes = {}, 0
                cur[k] = cpu(v)
                cur_bytes += nb
            if cur:
                shards.append(cur)
        else:
            n_slices = 16 + (1 if cfg.num_layers % 10 and cfg.num_layers >= 10 else 0)
            shards = [dict() for _ in range(n_slices)]
            for k, v in dense.items():
                shards[min(_dense_slice_of(k, cfg.num_layers), n_slices) - 1][k] = cpu(v)
        for i, sh in enumerate(shards):
            name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            save_file(sh, str(out / name), metadata={"format": "pt"})
            weight_map.update({k: name for k in sh})
    if experts:
        if ep > 1:
            name = f"moemodel-ep{store.ep_rank + 1:05d}-of-{ep:05d}.safetensors"
            save_file({k: cpu(v) for k, v in experts.items()}, str(out / name), metadata={"format": "pt"})
            mine = {k: name for k in experts}
            if _is_dist():
                maps = [None] * dist.get_world_size(group)
                dist.all_gather_object(maps, mine, group=group)
                for m in maps:
                    weight_map.update(m)
            else:
                weight_map.update(mine)
        elif rank == 0:
            for l in range(cfg.num_layers):
                name = f"moemodel-{l + 1:05d}-of-{cfg.num_layers:05d}.safetensors"
                part = {k: cpu(v) for k, v in experts.items() if f".layers.{l}." in k}
                save_file(part, str(out / name), metadata={"format": "pt"})
                weight_map.update({k: name for k in part})
    if rank == 0:
        total = sum(v.numel() * v.element_size() for v in sd.values())
        (out / "model.safetensors.index.json").write_text(
            json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}, indent=1))
        (out / "config.json").write_text(json.dumps(hf_config_dict(cfg), indent=1))
    if _is_dist():
        dist.barrier(group=group)
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
