"""Training configuration: a Python file evaluated into a dict-with-attributes, with the
same top-level keys, environment knobs and defaulting rules as the reference
(training/sensenovalm/core/context/parallel_context.py:51-139 ``Config``,
training/sensenovalm/initialize/launch.py:69-691 ``args_sanity_check``), and typed views
of it for the rest of this framework (ModelConfig, AdamConfig, ParallelConfig)."""
from __future__ import annotations

import contextlib
import importlib.util
import os
import runpy
import sys
import types
from typing import Any, Dict

import torch

from ..config import ModelConfig
from ..parallel.context import ParallelConfig
from .optimizer import AdamConfig


def env_bool(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    if v is None:
        return default
    return str(v).strip().lower() in ("1", "true", "yes", "y", "on")


@contextlib.contextmanager
def _config_helper_modules():
    """The reference's config files start with ``from sensenovalm.utils.config_helpers import env_bool``
    (training/configs/sensenovavl_qwen3_gen/sensenovau1_8b_mot_sft.py:7).  While a config file is evaluated, that
    module path resolves to this module's :func:`env_bool` unless the reference package itself is importable, so the
    reference's own config files load unchanged."""
    names = ("sensenovalm", "sensenovalm.utils", "sensenovalm.utils.config_helpers")
    try:
        have = importlib.util.find_spec("sensenovalm") is not None
    except (ImportError, ValueError):
        have = False
    if have or any(n in sys.modules for n in names):
        yield
        return
    mods = {n: types.ModuleType(n) for n in names}
    mods[names[0]].__path__ = []
    mods[names[1]].__path__ = []
    mods[names[0]].utils = mods[names[1]]
    mods[names[1]].config_helpers = mods[names[2]]
    mods[names[2]].env_bool = env_bool
    sys.modules.update(mods)
    try:
        yield
    finally:
        for n in names:
            sys.modules.pop(n, None)


class Config(dict):
    """dict whose items are also attributes; nested dicts are converted on the way in."""

    def __init__(self, d: Dict[str, Any] = None):
        super().__init__()
        for k, v in (d or {}).items():
            self[k] = v

    def __setitem__(self, k, v):
        if isinstance(v, dict) and not isinstance(v, Config):
            v = Config(v)
        super().__setitem__(k, v)

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e

    def __setattr__(self, k, v):
        self[k] = v

    @classmethod
    def from_file(cls, path: str) -> "Config":
        if not os.path.exists(path):
            raise FileNotFoundError(f"config file {path} not found")
        with _config_helper_modules():
            ns = runpy.run_path(path)
        return cls({k: v for k, v in ns.items() if not k.startswith("_") and not callable(v)
                    and not isinstance(v, type(os))})


_DTYPES = {"torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16, "torch.half": torch.float16,
           "torch.float32": torch.float32, "torch.tf32": torch.float32}


def sanity_check(cfg: Config, world_size: int = 1) -> Config:
    """Fills defaults and validates, following the reference's rules."""
    par = cfg.setdefault("parallel", Config())
    if not isinstance(par, Config):
        par = cfg["parallel"] = Config(par)

    def norm(key, default):
        v = par.get(key, None)
        if v is None:
            par[key] = Config(default)
        elif isinstance(v, int):
            d = dict(default); d["size"] = v
            par[key] = Config(d)
        else:
            for k, dv in default.items():
                v.setdefault(k, dv)
    norm("zero1", dict(size=-1, fsdp=False))
    norm("pipeline", dict(size=1, interleaved_overlap=False, zero_bubble=False))
    norm("tensor", dict(size=1, mode="mtp"))
    norm("weight", dict(size=1, overlap=False, launch_allgather_before="wo", forward_overlap_per="layer"))
    norm("expert", dict(size=-1, no_tp=False))
    norm("expert_weight", dict(size=1, overlap=False))
    if par.tensor.mode not in ("mtp", "msp", "fsp", "isp"):
        raise ValueError(f"parallel.tensor.mode {par.tensor.mode!r} must be one of mtp, msp, fsp, isp")
    if par.weight.size > 1 and par.tensor.mode != "isp":
        raise ValueError("parallel.weight.size > 1 requires parallel.tensor.mode == 'isp'")
    if par.pipeline.zero_bubble and par.pipeline.interleaved_overlap:
        raise ValueError("zero-bubble pipeline cannot be combined with interleaved overlap")
    if par.zero1.fsdp and (par.pipeline.size > 1 or par.tensor.mode == "isp"):
        raise ValueError("FSDP mode forbids pipeline parallel and ISP")
    model = cfg.setdefault("model", Config())
    if isinstance(model.get("dtype", "torch.float16"), str):
        name = model.get("dtype", "torch.float16")
        if name not in _DTYPES:
            raise ValueError(f"unknown model.dtype {name}")
        model["dtype"] = _DTYPES[name]
    ck = model.get("checkpoint", False)
    model["checkpoint"] = float(ck) if not isinstance(ck, bool) else (1.0 if ck else 0.0)
    if not 0.0 <= model["checkpoint"] <= 1.0:
        raise ValueError("model.checkpoint must be a bool or a fraction in [0, 1]")
    vocab = model.get("vocab_size")
    if vocab and (vocab % max(par.weight.size, 1) or vocab % max(par.tensor.size, 1)):
        raise ValueError("vocab_size must be divisible by the weight- and tensor-parallel sizes")
    moe = model.get("moe_kwargs") or {}
    is_moe = "MoE" in str(cfg.get("model_type", "")) and int(moe.get("num_experts", 1) or 1) > 1
    if par.expert.size in (-1, 0):
        par.expert["size"] = 1 if not is_moe else min(world_size, int(moe.get("num_experts", 1)))
    if not is_moe and (par.expert.size > 1 or par.expert_weight.size > 1):
        raise ValueError("expert / expert_weight parallel sizes > 1 need an MoE model")
    data = cfg.setdefault("data", Config())
    data.setdefault("micro_num", 1)
    data.setdefault("micro_bsz", 1)
    data.setdefault("valid_every", 0)
    data.setdefault("empty_cache_and_diag_interval", 50)
    data.setdefault("use_packed_dataset", True)
    if par.pipeline.size == 1:
        data["gradient_accumulation"] = data["micro_num"]
    ckpt = cfg.setdefault("ckpt", Config())
    ckpt.setdefault("enable_save_ckpt", True)
    if ckpt.enable_save_ckpt:
        if not ckpt.get("save_ckpt_folder") or int(ckpt.get("checkpoint_every", 0)) <= 0:
            raise ValueError("ckpt.enable_save_ckpt needs save_ckpt_folder and checkpoint_every > 0")
    ckpt.setdefault("auto_resume", True)
    ckpt.setdefault("oss_snapshot_freq", float("inf"))
    ckpt.setdefault("stop_file_path", None)
    hz = cfg.setdefault("hybrid_zero_optimizer", Config())
    hz.setdefault("overlap_sync_grad", False)
    hz.setdefault("overlap_sync_param", False)
    hz.setdefault("clip_grad_norm", 0)
    cfg.setdefault("reduce_comm_dtype", model["dtype"])
    from .config_check import check_sections
    cfg["_notes"] = check_sections(cfg)          # raises on settings this package does not implement
    return cfg


def model_config_from(cfg: Config, **overrides) -> ModelConfig:
    m = cfg.model
    moe = m.get("moe_kwargs") or {}
    hidden = int(m.hidden_size)
    kw = dict(name=cfg.get("JOB_NAME", "sft"), vocab_size=int(m.vocab_size), hidden_size=hidden,
              num_heads=int(m.num_attention_heads), num_kv_heads=int(m.num_kv_attention_heads),
              head_dim=int(m.get("head_dim", hidden // int(m.num_attention_heads))),
              ffn_size=int(round(hidden * float(m.get("mlp_ratio", 3.0)))), num_layers=int(m.num_layers),
              rms_eps=float(m.get("layer_norm_epsilon", 1e-6)), rope_base=float(m.get("rope_base", 5e6)),
              max_position_embeddings=int(m.get("max_position_embeddings", 262144)))
    if int(moe.get("num_experts", 0) or 0) > 1:
        kw.update(num_experts=int(moe["num_experts"]), num_experts_per_tok=int(moe.get("top_k", 1)),
                  gen_num_experts=int(moe.get("gen_num_experts", moe["num_experts"])),
                  gen_num_experts_per_tok=int(moe.get("gen_top_k", moe.get("top_k", 1))),
                  moe_intermediate_size=int(moe.get("moe_intermediate_size", kw["ffn_size"])),
                  router_aux_loss_coef=float((cfg.get("loss") or {}).get("expert_balance_coef", 0.0)),
                  router_z_loss_coef=float((cfg.get("loss") or {}).get("moe_z_loss_coef", 0.0)),
                  moe_balance_image_ratio=float(cfg.get("moe_balance_image_ratio", 0.0)),
                  moe_balance_text_ratio=float(cfg.get("moe_balance_text_ratio", 0.0)),
                  moe_balance_gen_ratio=float(cfg.get("moe_balance_gen_ratio", 1.0)),
                  moe_balance_und_ratio=float(cfg.get("moe_balance_und_ratio", 1.0)),
                  router_bias_update_rate=float(moe.get("aux_free_bias_update_rate", moe.get("bias_update_rate", 0.0)) or 0.0))
    for k in ("P_mean", "P_std", "time_schedule", "time_shift_type", "base_shift", "max_shift",
              "base_image_seq_len", "max_image_seq_len", "noise_scale_mode", "noise_scale",
              "noise_scale_base_image_seq_len", "noise_scale_max_value", "add_noise_scale_embedding", "t_eps",
              "use_pixel_head", "pixel_head_dim", "num_mtp_layers"):
        if k in m:
            kw[k] = m[k]
    if "ce_loss_weight" in cfg:
        kw["ce_loss_weight"] = float(cfg.ce_loss_weight)
    loss = cfg.get("loss") or {}
    if "image_gen_loss_coef" in loss:
        kw["image_gen_loss_weight"] = float(loss["image_gen_loss_coef"])
    kw.update(overrides)
    return ModelConfig(**kw)


def adam_config_from(cfg: Config) -> AdamConfig:
    a = cfg.get("adam") or {}
    ls = cfg.get("lr_scale") or {}
    return AdamConfig(lr=float(a.get("lr", 1e-4)), beta1=float(a.get("adam_beta1", 0.9)),
                      beta2=float(a.get("adam_beta2", 0.95)), eps=float(a.get("adam_eps", 1e-8)),
                      weight_decay=float(a.get("weight_decay", 0.0)),
                      clip_grad_norm=float((cfg.get("hybrid_zero_optimizer") or {}).get("clip_grad_norm", 0)),
                      lr_scale={"vit": float(ls.get("mlp_lr_scale", 1.0)),
                                "fm_modules": float(ls.get("fm_modules_lr_scale", 1.0)),
                                "moe_gate": float(ls.get("moe_wg_lr_scale", 1.0)),
                                "mot_gen": float(ls.get("mot_gen_lr_scale", 1.0))})


def parallel_config_from(cfg: Config) -> ParallelConfig:
    return ParallelConfig.from_dict(cfg.parallel)
