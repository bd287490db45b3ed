"""Local (in-process) model for the ComfyUI nodes: loading, a one-entry model cache with eviction,
memory logging and the three generation tasks on this framework's ``NEOChatModel``.

Covers the role of the reference's apps/comfyui/local_pipeline.py:211-580 (model wrapper and task
methods) and nodes.py:181-215 (cache eviction); the sampling itself is
``sensenova_u1_b200.inference``.
"""
from __future__ import annotations

import gc
import logging
import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

LOGGER = logging.getLogger("sensenova_u1_b200.comfyui")
VRAM_MODES = ("full", "fast", "balanced", "low")
CFG_NORMS = ("none", "global", "channel", "cfg_zero_star")
IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)


def memory_report(device=None) -> str:
    if not torch.cuda.is_available():
        return "cuda unavailable"
    free, total = torch.cuda.mem_get_info(device)
    return (f"allocated {torch.cuda.memory_allocated(device) / 2**30:.2f} GiB, reserved "
            f"{torch.cuda.memory_reserved(device) / 2**30:.2f} GiB, free {free / 2**30:.2f} of {total / 2**30:.2f} GiB")


def snap_size(width: int, height: int, factor: int = 32, min_side: int = 64) -> Tuple[int, int]:
    """Image sides as multiples of the token size (32 pixels for every released model)."""
    snap = lambda v: max(min_side, int(round(v / factor)) * factor)
    return snap(width), snap(height)


@dataclass
class LocalModel:
    model: object
    tokenizer: object
    key: tuple
    device: str = "cuda"

    @property
    def token_pixels(self) -> int:
        return int(getattr(getattr(self.model, "cfg", None), "token_pixels", 32))

    # -- tasks ---------------------------------------------------------------------------------
    def text_to_image(self, prompt: str, width: int, height: int, steps: int = 50, cfg_scale: float = 4.0,
                      timestep_shift: float = 3.0, cfg_norm: str = "none", seed: int = 0, batch_size: int = 1,
                      think: bool = False) -> Tuple[torch.Tensor, str]:
        w, h = snap_size(width, height, self.token_pixels)
        out = self.model.t2i_generate(self.tokenizer, prompt, cfg_scale=cfg_scale, timestep_shift=timestep_shift,
                                      cfg_norm=cfg_norm, image_size=(w, h), num_steps=steps, batch_size=batch_size,
                                      think_mode=think, seed=seed)
        imgs, thought = (out if think else (out, ""))
        LOGGER.info("t2i %dx%d, %d steps: %s", w, h, steps, memory_report())
        return imgs, thought

    def _as_understanding_inputs(self, images: Sequence[torch.Tensor], max_side: int) -> List[torch.Tensor]:
        """[-1,1] pictures -> ImageNet-normalised, sides snapped to the token size and bounded."""
        mean = torch.tensor(IMAGENET_MEAN).view(3, 1, 1)
        std = torch.tensor(IMAGENET_STD).view(3, 1, 1)
        out = []
        for im in images:
            _, H, W = im.shape
            scale = min(1.0, max_side / max(H, W))
            w, h = snap_size(W * scale, H * scale, self.token_pixels)
            if (h, w) != (H, W):
                im = torch.nn.functional.interpolate(im[None].float(), size=(h, w), mode="bicubic",
                                                     align_corners=False)[0]
            out.append(((im.float().clamp(-1, 1) * 0.5 + 0.5) - mean) / std)
        return out

    def edit_image(self, prompt: str, images: Sequence[torch.Tensor], steps: int = 50, cfg_scale: float = 4.0,
                   img_cfg_scale: float = 1.0, timestep_shift: float = 3.0, cfg_norm: str = "none", seed: int = 0,
                   width: int = 0, height: int = 0, max_side: int = 2048) -> torch.Tensor:
        if not images:
            raise ValueError("image editing needs at least one input image")
        und = self._as_understanding_inputs(images, max_side)
        size = snap_size(width, height, self.token_pixels) if width > 0 and height > 0 else None
        out = self.model.it2i_generate(self.tokenizer, prompt, und, cfg_scale=cfg_scale, img_cfg_scale=img_cfg_scale,
                                       timestep_shift=timestep_shift, cfg_norm=cfg_norm, image_size=size,
                                       num_steps=steps, seed=seed)
        LOGGER.info("edit, %d input image(s), %d steps: %s", len(images), steps, memory_report())
        return out

    def interleave(self, prompt: str, images: Sequence[torch.Tensor] = (), width: int = 1024, height: int = 1024,
                   steps: int = 50, cfg_scale: float = 4.0, timestep_shift: float = 3.0, seed: int = 0,
                   max_rounds: int = 4, max_new_tokens: int = 512, max_side: int = 2048):
        und = self._as_understanding_inputs(images, max_side)
        text, imgs = self.model.interleave_gen(self.tokenizer, prompt, und, max_rounds=max_rounds,
                                               max_new_tokens=max_new_tokens,
                                               image_size=snap_size(width, height, self.token_pixels),
                                               cfg_scale=cfg_scale, timestep_shift=timestep_shift, num_steps=steps,
                                               seed=seed)
        LOGGER.info("interleave, %d picture(s): %s", len(imgs), memory_report())
        return text, list(imgs)


# ------------------------------------------------------------------------------------------------
# one resident model at a time: loading another one first releases the old one's device and pinned memory
# ------------------------------------------------------------------------------------------------
_CACHE: Dict[tuple, LocalModel] = {}


def evict(keep: Optional[tuple] = None) -> int:
    drop = [k for k in _CACHE if k != keep]
    for k in drop:
        lm = _CACHE.pop(k)
        lm.model = None
        lm.tokenizer = None
    if drop:
        gc.collect()                       # cycles must be gone before the allocator can return the blocks
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
            empty_host = getattr(torch._C, "_host_emptyCache", None)
            if empty_host is not None:     # pinned staging of an offloaded model
                empty_host()
        LOGGER.info("evicted %d cached model(s): %s", len(drop), memory_report())
    return len(drop)


def _default_loader(model_path: str, device: str, vram_mode: str, gguf: str, random_init: str, dtype: str = "bfloat16",
                    max_memory: str = "", offload_kwargs: Optional[dict] = None):
    import sensenova_u1_b200 as pkg
    from sensenova_u1_b200.inference.api import ByteTokenizer
    dt = getattr(torch, dtype)
    if random_init:
        from sensenova_u1_b200.config import get_config
        kw = {"head_dim": 128} if random_init == "tiny-mot" else {}
        cfg = get_config(random_init, **kw)
        model = pkg.NEOChatModel.from_config(cfg, device=device, vram_mode=vram_mode, dtype=dt, offload_kwargs=offload_kwargs)
        return model, ByteTokenizer(cfg.vocab_size)
    caps = parse_max_memory(max_memory)
    model = pkg.NEOChatModel.from_pretrained(model_path, device_map=device, torch_dtype=dt, max_memory=caps or None,
                                             vram_mode=None if (caps and vram_mode == "full") else vram_mode,
                                             offload_kwargs=offload_kwargs)
    if gguf:
        from sensenova_u1_b200.utils.gguf_loader import load_gguf
        load_gguf(gguf, model.store)
    from transformers import AutoTokenizer
    return model, AutoTokenizer.from_pretrained(model_path, trust_remote_code=False)


def parse_max_memory(text: str) -> Dict:
    """``"0=20GiB,cpu=64GiB"`` -> ``{0: "20GiB", "cpu": "64GiB"}`` (the loader node's text field)."""
    out: Dict = {}
    for part in (text or "").replace(";", ",").split(","):
        part = part.strip()
        if not part:
            continue
        if "=" not in part:
            raise ValueError(f"max_memory entries look like 0=20GiB or cpu=64GiB, got {part!r}")
        k, v = (x.strip() for x in part.split("=", 1))
        out[int(k) if k.isdigit() else k] = v
    return out


def fast_offload_kwargs(device: str, vram_mode: str, fraction: float = 0.9, headroom_gib: float = 2.0,
                        activation_reserve_gib: float = 4.0, budget_gib: float = 0.0, mem_info=None) -> Optional[dict]:
    """Explicit residency budget of the "fast" mode from the loader node's advanced fields; None for the other modes
    (their presets apply)."""
    if vram_mode != "fast":
        return None
    from sensenova_u1_b200.utils.offload import fast_mode_budget
    return {"resident_budget_bytes": fast_mode_budget(device, fraction, headroom_gib, activation_reserve_gib, budget_gib,
                                                      mem_info=mem_info)}


def load(model_path: str, device: str = "cuda", vram_mode: str = "full", gguf: str = "", random_init: str = "",
         loader: Optional[Callable] = None, dtype: str = "bfloat16", max_memory: str = "",
         offload_kwargs: Optional[dict] = None) -> LocalModel:
    """Returns the cached model for these settings or loads it (evicting any other)."""
    if vram_mode not in VRAM_MODES:
        raise ValueError(f"vram_mode must be one of {VRAM_MODES}")
    if dtype not in ("bfloat16", "float16", "float32"):
        raise ValueError("dtype must be bfloat16, float16 or float32")
    key = (os.path.abspath(model_path) if os.path.exists(model_path) else model_path, device, vram_mode, gguf,
           random_init, dtype, max_memory, tuple(sorted((offload_kwargs or {}).items())))
    if key in _CACHE:
        return _CACHE[key]
    evict(keep=None)
    if loader is not None:
        model, tok = loader(model_path, device, vram_mode, gguf, random_init)
    else:
        model, tok = _default_loader(model_path, device, vram_mode, gguf, random_init, dtype, max_memory, offload_kwargs)
    _CACHE[key] = LocalModel(model, tok, key, device)
    LOGGER.info("loaded %s (%s): %s", model_path or random_init, vram_mode, memory_report())
    return _CACHE[key]
