"""Helpers around the model: loading, offload, profiling, LoRA / GGUF, parameter report, picture comparison.

The names the reference exports from ``sensenova_u1.utils`` (src/sensenova_u1/utils/__init__.py:1-80) resolve here as
well, each to this package's implementation, so scripts written against the reference keep their imports.  Everything
is imported on first use: ``import sensenova_u1_b200.utils`` stays light."""
from __future__ import annotations

import importlib

DEFAULT_VRAM_MODE = "full"
VRAM_MODE_OPTIONS = ("full", "fast", "balanced", "low")
DEFAULT_FAST_VRAM_FRACTION = 0.9
DEFAULT_FAST_VRAM_HEADROOM_GIB = 2.0
DEFAULT_FAST_ACTIVATION_RESERVE_GIB = 4.0
DEFAULT_IMAGE_PATCH_SIZE = 32            # side of one image token in pixels (profiler's tokens-per-second figure)

# exported name -> (module, attribute)
_LAZY = {
    "InferenceProfiler": ("profiler", "InferenceProfiler"),
    "LayerOffloader": ("offload", "LayerOffloader"),
    "vram_mode_for_budget": ("offload", "vram_mode_for_budget"),
    "fast_mode_budget": ("offload", "fast_mode_budget"),
    "parse_max_memory": ("cli", "parse_max_memory"),
    "add_offload_args": ("cli", "add_model_args"),          # model + memory flags are one argument group set here
    "save_compare": ("comparison", "comparison_sheet"),
    "comparison_sheet": ("comparison", "comparison_sheet"),
    "load_gguf_checkpoint": ("gguf_loader", "load_gguf"),
    "merge_lora": ("lora", "merge_lora"),
    "load_lora_state": ("cli", "load_lora_state"),
    "breakdown": ("param_count", "breakdown"),
    "inspect_checkpoint": ("param_count", "inspect_checkpoint"),
    "build_rules": ("param_count", "load_rules"),
    "format_param_count": ("param_count", "si"),
    "MemoryWatch": ("diagnostics", "MemoryWatch"),
    "check_replicas_equal": ("diagnostics", "check_replicas_equal"),
}


def load_model_and_tokenizer(*a, **kw):
    """(model, tokenizer) from a checkpoint directory or hub id (``device_map``, ``max_memory``, ``vram_mode``)."""
    from ..inference.hf import load_model_and_tokenizer as f
    return f(*a, **kw)


def load_and_merge_lora_weight_from_safetensors(model, lora_path: str, alpha=None, scale: float = 1.0) -> int:
    """Merges LoRA pairs (``up @ down * alpha / rank``) from a file or folder into the model's weights; returns the
    number of merged pairs."""
    from .cli import load_lora_state
    from .lora import merge_lora
    return merge_lora(getattr(model, "store", model), load_lora_state(lora_path), alpha=alpha, scale=scale)


def best_available_device() -> str:
    import torch
    return "cuda" if torch.cuda.is_available() else "cpu"


def seed_all_accelerators(seed: int) -> None:
    import torch
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def infer_input_device(model):
    """Device the model's inputs go to."""
    store = getattr(model, "store", None)
    if store is not None:
        return store.device
    impl = getattr(model, "impl", None)
    return impl.store.device if impl is not None else next(model.parameters()).device


def format_bytes(n: int) -> str:
    from .param_count import si
    return si(n, (("GB", 1e9), ("MB", 1e6), ("KB", 1e3))) if abs(n) >= 1e3 else f"{int(n)}B"


def vram_mode_keeps_generation_resident(mode: str) -> bool:
    """``fast`` keeps the generation halves of streamed layers on the device during denoising."""
    from .offload import VRAM_MODES
    return float(VRAM_MODES[mode].get("gen_resident", 0.0) or 0.0) > 0.0


def vram_mode_to_prefetch_count(mode: str) -> int:
    from .offload import VRAM_MODES
    return int(VRAM_MODES[mode].get("prefetch", 0) or 0)


def __getattr__(name: str):
    if name in _LAZY:
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = sorted(list(_LAZY) + [
    "DEFAULT_VRAM_MODE", "VRAM_MODE_OPTIONS", "DEFAULT_FAST_VRAM_FRACTION", "DEFAULT_FAST_VRAM_HEADROOM_GIB",
    "DEFAULT_FAST_ACTIVATION_RESERVE_GIB", "DEFAULT_IMAGE_PATCH_SIZE", "load_model_and_tokenizer",
    "load_and_merge_lora_weight_from_safetensors", "best_available_device", "seed_all_accelerators", "infer_input_device",
    "format_bytes", "vram_mode_keeps_generation_resident", "vram_mode_to_prefetch_count"])
