"""Hugging Face integration of the inference model: ``transformers`` configuration classes,
``AutoConfig`` / ``AutoModel`` registration and a ``PreTrainedModel``-shaped loader, with the reference's
names (src/sensenova_u1/models/neo_unify/__init__.py:36-55, configuration_neo_chat.py:21-197,
configuration_neo_vit.py, modeling_neo_chat.py:151-170, utils/checkpoint_loading.py:182-247).

The model itself is this package's sm_100a inference engine.  Its weights live in the flat arenas of a
:class:`ParamStore`; the ``PreTrainedModel`` wrapper exposes them as parameters under the checkpoint's
key names (views into the arenas, no copies), so ``state_dict()``, ``named_parameters()``,
``num_parameters()`` and ``save_pretrained()`` behave as users of the reference expect, while
``from_pretrained`` streams safetensors shards straight into the arenas instead of building modules.

    from transformers import AutoConfig, AutoModel
    import sensenova_u1_b200                       # registers "neo_chat" / "neo_vision"
    model = AutoModel.from_pretrained(path, torch_dtype=torch.bfloat16, device_map="cuda")
    image = model.t2i_generate(tokenizer, "a red bicycle", cfg_scale=4.0, image_size=(1024, 1024))
"""
from __future__ import annotations

import copy
import json
from pathlib import Path
from typing import Dict, Optional, Union

import torch
from torch import nn
from transformers import PretrainedConfig, PreTrainedModel, Qwen3Config, Qwen3MoeConfig

from ..config import ModelConfig
from ..models.params import ParamStore, hf_state_dict
from . import api as _api


def _legacy_rope_theta(cfg) -> None:
    """transformers 5 moved ``rope_theta`` into ``rope_parameters``; the checkpoints carry the old field."""
    if not hasattr(cfg, "rope_theta") or cfg.rope_theta is None:
        rp = getattr(cfg, "rope_parameters", None) or {}
        cfg.rope_theta = float(rp.get("rope_theta", 10000.0))


class NEOVisionConfig(PretrainedConfig):
    model_type = "neo_vision"

    def __init__(self, num_channels=3, patch_size=16, hidden_size=1024, llm_hidden_size=2048, downsample_ratio=0.5,
                 rope_theta_vision=10000.0, max_position_embeddings_vision=10000, min_pixels=65536,
                 max_pixels=4194304, **kwargs):
        super().__init__(**kwargs)
        self.num_channels, self.patch_size, self.hidden_size = num_channels, patch_size, hidden_size
        self.llm_hidden_size, self.downsample_ratio = llm_hidden_size, downsample_ratio
        self.rope_theta_vision = rope_theta_vision
        self.max_position_embeddings_vision = max_position_embeddings_vision
        self.min_pixels, self.max_pixels = min_pixels, max_pixels


class NEOLLMConfig(Qwen3Config):
    """Dense backbone: ``Qwen3Config`` plus the rope base of the two spatial axes."""

    def __init__(self, rope_theta_hw=10000.0, max_position_embeddings_hw=10000, **kwargs):
        super().__init__(**kwargs)
        _legacy_rope_theta(self)
        self.rope_theta_hw, self.max_position_embeddings_hw = rope_theta_hw, max_position_embeddings_hw


class NEOMoELLMConfig(Qwen3MoeConfig):
    """Mixture-of-experts backbone: ``Qwen3MoeConfig`` plus the generation branch's own mixture; every
    ``gen_*`` knob falls back to the understanding branch's value."""

    def __init__(self, rope_theta_hw=10000.0, max_position_embeddings_hw=10000, gen_num_experts=None,
                 gen_num_experts_per_tok=None, gen_moe_intermediate_size=None, **kwargs):
        super().__init__(**kwargs)
        _legacy_rope_theta(self)
        self.rope_theta_hw, self.max_position_embeddings_hw = rope_theta_hw, max_position_embeddings_hw
        self.gen_num_experts = int(self.num_experts if gen_num_experts is None else gen_num_experts)
        self.gen_num_experts_per_tok = int(self.num_experts_per_tok if gen_num_experts_per_tok is None
                                           else gen_num_experts_per_tok)
        self.gen_moe_intermediate_size = int(self.moe_intermediate_size if gen_moe_intermediate_size is None
                                             else gen_moe_intermediate_size)


def _is_moe(llm) -> bool:
    get = (lambda k, d=None: llm.get(k, d)) if isinstance(llm, dict) else (lambda k, d=None: getattr(llm, k, d))
    if "moe" in str(get("model_type", "")).lower():
        return True
    if any("moe" in str(a).lower() for a in (get("architectures") or [])):
        return True
    return int(get("num_experts", 0) or 0) > 1


_FLOW_KEYS = dict(noise_scale=1.0, noise_scale_mode="resolution", noise_scale_base_image_seq_len=64,
                  noise_scale_max_value=8.0, add_noise_scale_embedding=True, t_eps=0.05, time_schedule="standard",
                  time_shift_type="exponential", base_shift=0.5, max_shift=1.15, base_image_seq_len=64,
                  max_image_seq_len=4096, use_pixel_head=False, fm_head_dim=4096, fm_head_layers=2,
                  fm_head_mlp_ratio=1, concat_time_token_num=0)


class NEOChatConfig(PretrainedConfig):
    model_type = "neo_chat"
    is_composition = True

    def __init__(self, vision_config=None, llm_config=None, use_backbone_lora=0, use_llm_lora=0, downsample_ratio=0.5,
                 template=None, **kwargs):
        flow = {k: kwargs.pop(k, d) for k, d in _FLOW_KEYS.items()}
        super().__init__(**kwargs)
        vision_config = {"architectures": ["NEOVisionModel"]} if vision_config is None else vision_config
        llm_config = {"architectures": ["Qwen3ForCausalLM"]} if llm_config is None else llm_config
        self.vision_config = NEOVisionConfig(**vision_config) if isinstance(vision_config, dict) else vision_config
        if isinstance(llm_config, dict):
            llm_config = (NEOMoELLMConfig if _is_moe(llm_config) else NEOLLMConfig)(**llm_config)
        self.llm_config = llm_config
        self.use_backbone_lora, self.use_llm_lora = use_backbone_lora, use_llm_lora
        self.downsample_ratio, self.template = downsample_ratio, template
        self.tie_word_embeddings = bool(getattr(self.llm_config, "tie_word_embeddings", False))
        for k, v in flow.items():
            setattr(self, k, v)

    @property
    def is_moe_llm(self) -> bool:
        return isinstance(self.llm_config, NEOMoELLMConfig)

    def to_dict(self):
        out = copy.deepcopy({k: v for k, v in self.__dict__.items() if k not in ("vision_config", "llm_config")})
        out["vision_config"] = self.vision_config.to_dict()
        out["llm_config"] = self.llm_config.to_dict()
        if "num_local_experts" in out["llm_config"] and "num_experts" not in out["llm_config"]:
            # transformers 5 serialises Qwen3-MoE's expert count under its new name; checkpoints carry the old one
            out["llm_config"]["num_experts"] = out["llm_config"]["num_local_experts"]
        out["model_type"] = self.model_type
        return out

    def to_model_config(self, **overrides) -> ModelConfig:
        from ..train.checkpoint import config_from_hf
        d = self.to_dict()
        llm = d["llm_config"]
        llm.setdefault("rope_theta", getattr(self.llm_config, "rope_theta", 5e6))
        return config_from_hf(d, **overrides)

    @classmethod
    def from_model_config(cls, cfg: ModelConfig) -> "NEOChatConfig":
        from ..train.checkpoint import hf_config_dict
        d = hf_config_dict(cfg)
        d.pop("model_type", None); d.pop("architectures", None)
        d["llm_config"]["architectures"] = ["Qwen3MoeForCausalLM" if cfg.is_moe else "Qwen3ForCausalLM"]
        return cls(**d)


class _Holder(nn.Module):
    """A node of the module tree that mirrors the checkpoint's key paths."""


def _attach(root: nn.Module, dotted: str, tensor: torch.Tensor) -> None:
    *path, leaf = dotted.split(".")
    mod = root
    for part in path:
        if part not in mod._modules:
            mod.add_module(part, _Holder())
        mod = mod._modules[part]
    mod.register_parameter(leaf, nn.Parameter(tensor, requires_grad=False))


class NEOChatModel(PreTrainedModel):
    """``PreTrainedModel`` face of the inference engine (reference: modeling_neo_chat.py:151-170).

    Generation entry points (``t2i_generate``, ``it2i_generate``, ``interleave_gen``,
    ``interleave_gen_image_only``, ``chat``, ``generate``) are those of :class:`inference.api.NEOChatModel`
    and run on the hand-written kernels; ``forward`` is not a training path here either (the reference's raises
    as well, modeling_neo_chat.py:272).
    """
    config_class = NEOChatConfig
    main_input_name = "pixel_values"
    base_model_prefix = "language_model"
    _supports_flash_attn_2 = True
    supports_gradient_checkpointing = False
    _no_split_modules = ["NEOVisionModel", "Qwen3DecoderLayer", "Qwen3MoeDecoderLayer"]
    _tp_plan = ""

    def __init__(self, config: NEOChatConfig, store: Optional[ParamStore] = None, vram_mode: str = "full",
                 device=None, dtype=torch.bfloat16, offload_kwargs: Optional[dict] = None):
        super().__init__(config)
        mcfg = config.to_model_config()
        if store is None:
            dev = device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu")
            store = ParamStore(mcfg, device=dev if vram_mode == "full" else "cpu", dtype=dtype, with_grads=False)
            store.init_weights(0)
        self.store = store
        for k, v in hf_state_dict(store).items():
            _attach(self, k, v)
        self._impl = None
        self._impl_args = (vram_mode, device, offload_kwargs)
        self.template = config.template
        self.patch_size = config.vision_config.patch_size
        self.downsample_ratio = config.downsample_ratio
        self.img_context_token_id = None
        self.img_start_token_id = 151670

    # the engine allocates device workspaces: built on first use, so that CPU-only tools (key listing, parameter
    # counts, save_pretrained) work without a GPU
    @property
    def impl(self) -> "_api.NEOChatModel":
        if self._impl is None:
            vram_mode, device, okw = self._impl_args
            self._impl = _api.NEOChatModel(self.store.cfg, self.store, vram_mode=vram_mode, device=device,
                                           offload_kwargs=okw)
        return self._impl

    def _init_weights(self, module):          # weights are initialised in the arenas
        return

    def forward(self, *args, **kwargs):
        raise NotImplementedError("forward: use t2i_generate / it2i_generate / interleave_gen / chat / generate")

    # ---- loading ------------------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: Union[str, Path], *model_args, config=None,
                        torch_dtype=None, dtype=None, device_map=None, max_memory: Optional[Dict] = None,
                        vram_mode: Optional[str] = None, local_files_only: bool = True,
                        offload_kwargs: Optional[dict] = None, **kwargs):
        """Loads a checkpoint directory (safetensors shards + config.json).  ``device_map``: None / "cpu" / "cuda" /
        "cuda:i" / "auto" / {"": device}.  ``max_memory`` (``{0: "20GiB", "cpu": ...}``, the reference's
        ``--max_memory`` caps, utils/checkpoint_loading.py:236-245) selects layer streaming from pinned host
        memory when the cap for the GPU is below the checkpoint's size; ``vram_mode`` picks the streaming depth
        directly."""
        from ..train.checkpoint import import_hf
        from ..utils.offload import vram_mode_for_budget
        path = Path(resolve_checkpoint_path(pretrained_model_name_or_path))
        raw = json.loads((path / "config.json").read_text())
        _api.check_checkpoint_compatibility(raw)
        if config is None:
            r = dict(raw); r.pop("model_type", None); r.pop("architectures", None)
            config = NEOChatConfig(**r)
        dt = dtype if dtype is not None else torch_dtype
        if isinstance(dt, str):
            dt = getattr(torch, dt.replace("torch.", ""))
        dt = dt or torch.bfloat16
        dev = device_map.get("", "cuda") if isinstance(device_map, dict) else device_map
        if dev in (None, "auto", "balanced", "sequential"):
            dev = "cuda" if torch.cuda.is_available() else "cpu"
        if vram_mode is None:
            vram_mode = "full"
            if max_memory:
                total = sum(f.stat().st_size for f in path.glob("*.safetensors"))
                vram_mode = vram_mode_for_budget(max_memory, total, torch.device(dev))
        store = import_hf(str(path), device=dev if vram_mode == "full" else "cpu", dtype=dt, with_grads=False)
        return cls(config, store=store, vram_mode=vram_mode, device=dev, dtype=dt, offload_kwargs=offload_kwargs)

    @classmethod
    def from_config(cls, cfg, device="cuda", seed: int = 0, vram_mode: str = "full", dtype=torch.bfloat16,
                    offload_kwargs: Optional[dict] = None):
        """Random-init model from this package's :class:`ModelConfig` or from a :class:`NEOChatConfig`."""
        config = cfg if isinstance(cfg, NEOChatConfig) else NEOChatConfig.from_model_config(cfg)
        mcfg = cfg if isinstance(cfg, ModelConfig) else config.to_model_config()
        store = ParamStore(mcfg, device=device if vram_mode == "full" else "cpu", dtype=dtype, with_grads=False)
        store.init_weights(seed)
        return cls(config, store=store, vram_mode=vram_mode, device=device, dtype=dtype, offload_kwargs=offload_kwargs)

    @property
    def cfg(self) -> ModelConfig:
        return self.store.cfg

    @property
    def engine(self):
        return self.impl.engine

    def enable_sequence_parallel(self, sp_group, par_group=None) -> None:
        self.impl.enable_sequence_parallel(sp_group, par_group)

    def save_pretrained(self, save_directory, **kwargs):
        from ..train.checkpoint import export_hf
        export_hf(self.store, str(save_directory), max_shard_bytes=kwargs.get("max_shard_bytes"))
        (Path(save_directory) / "config.json").write_text(json.dumps(self.config.to_dict(), indent=1, default=str))

    # ---- generation: the engine's entry points ----------------------------------------------------------------
    def t2i_generate(self, *a, **k):
        return self.impl.t2i_generate(*a, **k)

    def it2i_generate(self, *a, **k):
        return self.impl.it2i_generate(*a, **k)

    def interleave_gen(self, *a, **k):
        return self.impl.interleave_gen(*a, **k)

    def interleave_gen_image_only(self, *a, **k):
        return self.impl.interleave_gen_image_only(*a, **k)

    def chat(self, *a, **k):
        return self.impl.chat(*a, **k)

    def generate(self, *a, **k):
        return self.impl.generate(*a, **k)

    def batch_chat(self, *a, **k):
        return self.impl.batch_chat(*a, **k)

    def extract_feature(self, pixel_values, gen_model: bool = False, grid_hw=None):
        return self.impl.extract_feature(pixel_values, gen_model=gen_model, grid_hw=grid_hw)

    patchify = staticmethod(_api.NEOChatModel.patchify)
    unpatchify = staticmethod(_api.NEOChatModel.unpatchify)

    @property
    def lm_head(self):
        return self.get_output_embeddings()

    def get_input_embeddings(self):
        return self.language_model.model.embed_tokens

    def get_output_embeddings(self):
        return self.language_model.lm_head

    def get_thw_indexes(self, input_ids, grid_hw=None):
        """(t, h, w) index per token; ``grid_hw``: patch grids (before the 2x2 merge) as in the reference
        (modeling_neo_chat.py:1977-1992)."""
        m = int(round(1 / self.downsample_ratio))
        grids = [] if grid_hw is None else [(int(h) // m, int(w) // m) for h, w in torch.as_tensor(grid_hw).tolist()]
        return _api.NEOChatModel.get_thw_indexes(input_ids.cpu(), grids, self.img_context_token_id).to(torch.long)


def snapshot_is_complete(d: Path) -> bool:
    """A checkpoint directory with all of its weight files: one ``model.safetensors``, or an index whose every
    shard is present (a cache left by an interrupted download has the config and some shards only; reference:
    utils/checkpoint_loading.py:250-323, tests/test_checkpoint_loading.py)."""
    d = Path(d)
    index = d / "model.safetensors.index.json"
    if index.is_file():
        try:
            shards = set(json.loads(index.read_text())["weight_map"].values())
        except (OSError, ValueError, KeyError):
            return False
        return bool(shards) and all((d / s).is_file() for s in shards)
    return (d / "model.safetensors").is_file() or any(d.glob("*.safetensors"))


def resolve_checkpoint_path(name_or_path: Union[str, Path]) -> str:
    """A local directory as given; otherwise the newest snapshot of that repository id in the local Hugging Face
    cache (offline resolution, utils/checkpoint_loading.py:250-323).  Nothing is downloaded."""
    p = Path(str(name_or_path)).expanduser()
    if p.is_dir():
        return str(p)
    import os
    cache = Path(os.environ.get("HF_HUB_CACHE") or Path(os.environ.get("HF_HOME", Path.home() / ".cache" / "huggingface")) / "hub")
    repo = cache / ("models--" + str(name_or_path).replace("/", "--")) / "snapshots"
    if repo.is_dir():
        snaps = sorted((d for d in repo.iterdir() if (d / "config.json").exists()), key=lambda d: d.stat().st_mtime)
        whole = [d for d in snaps if snapshot_is_complete(d)]
        if whole:
            return str(whole[-1])
        if snaps:
            raise FileNotFoundError(f"the cached snapshot of {name_or_path!r} ({snaps[-1]}) is missing weight files "
                                    f"(an interrupted download); this build does not download")
    raise FileNotFoundError(f"{name_or_path!r} is neither a checkpoint directory nor a repository in the local "
                            f"Hugging Face cache ({cache}); this build does not download")


def load_model_and_tokenizer(model_path: str, device: str = "cuda", dtype=torch.bfloat16, device_map=None,
                             max_memory=None, vram_mode: Optional[str] = None, tokenizer=None, **kw):
    """(model, tokenizer) for the example CLIs (reference: utils/checkpoint_loading.py:182-247)."""
    model = NEOChatModel.from_pretrained(model_path, dtype=dtype, device_map=device_map or device,
                                         max_memory=max_memory, vram_mode=vram_mode)
    if tokenizer is None:
        try:
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(resolve_checkpoint_path(model_path), trust_remote_code=False)
        except Exception:            # a checkpoint directory without tokenizer files (synthetic tests)
            tokenizer = _api.ByteTokenizer(model.store.cfg.vocab_size)
    return model, tokenizer


def register() -> None:
    """Registers the configuration and model classes with ``AutoConfig`` / ``AutoModel`` (idempotent)."""
    from transformers import AutoConfig, AutoModel
    for name, c in (("neo_vision", NEOVisionConfig), ("neo_chat", NEOChatConfig)):
        try:
            AutoConfig.register(name, c)
        except ValueError:
            pass
    try:
        AutoModel.register(NEOChatConfig, NEOChatModel)
    except ValueError:
        pass
