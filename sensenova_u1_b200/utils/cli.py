"""Shared pieces of the example command lines (examples/{t2i,editing,interleave,vqa}/inference.py).

The flags are the reference's (examples/t2i/inference.py:196-348, examples/editing/inference.py:204-360,
examples/interleave/inference.py:131-260, examples/vqa/inference.py:29-112 and the loader / offload flags of
src/sensenova_u1/utils/checkpoint_loading.py:49-179), plus ``--random_init`` / ``--layers`` to run without a
checkpoint.  ``--attn_backend`` is accepted for compatibility: attention always runs on this package's kernel.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path
from typing import Any, Dict, Iterator, List, Optional, Sequence, Tuple

VRAM_MODES = ("full", "fast", "balanced", "low")
CFG_NORMS = ("none", "global", "channel", "cfg_zero_star")
DTYPES = ("bfloat16", "float16", "float32")
# resolution buckets the released checkpoints were trained on (examples/t2i/inference.py:35-47)
SUPPORTED_RESOLUTIONS = ((2048, 2048), (2752, 1536), (1536, 2752), (2496, 1664), (1664, 2496), (2368, 1760), (1760, 2368),
                         (2272, 1824), (1824, 2272), (3072, 1376), (1344, 3136))


# ---------------------------------------------------------------------------------------------------------------
# argument groups
# ---------------------------------------------------------------------------------------------------------------
def add_model_args(p: argparse.ArgumentParser) -> None:
    g = p.add_argument_group("model")
    g.add_argument("--model_path", default=None, help="Hugging Face id with a complete local snapshot, or a checkpoint directory")
    g.add_argument("--random_init", default=None, help="model preset for a run without a checkpoint (tiny-mot, 8b-mot, a3b-mot)")
    g.add_argument("--layers", type=int, default=None, help="with --random_init: override the layer count")
    g.add_argument("--lora_path", default=None, help="LoRA weights (safetensors / .pt) merged into the base weights at load")
    g.add_argument("--gguf_checkpoint", default=None, help=".gguf file whose tensors replace the checkpoint's (de-quantised at load)")
    g.add_argument("--device", default="cuda", help="compute device, e.g. cuda or cuda:0")
    g.add_argument("--dtype", default="bfloat16", choices=DTYPES)
    g.add_argument("--attn_backend", default="auto", choices=["auto", "flash", "sdpa", "sm100"],
                   help="accepted for compatibility; attention runs on this package's sm_100a kernel")
    o = p.add_argument_group("memory")
    o.add_argument("--vram_mode", default="full", choices=VRAM_MODES,
                   help="full: all weights resident; fast / balanced / low: decoder layers stream from pinned host memory")
    o.add_argument("--device_map", default="none", help="none | auto | cuda:i (one device per process in this package)")
    o.add_argument("--max_memory", default="", help='per-device caps, e.g. "0=20GiB,cpu=64GiB": picks a streaming mode that fits')
    o.add_argument("--fast_vram_fraction", type=float, default=0.9)
    o.add_argument("--fast_vram_headroom_gib", type=float, default=2.0)
    o.add_argument("--fast_activation_reserve_gib", type=float, default=4.0)
    o.add_argument("--fast_vram_budget_gib", type=float, default=0.0, help="explicit residency budget of the fast mode (0: automatic)")
    p.add_argument("--profile", action="store_true", help="print load time, time per call, image tokens per second, peak memory")


def add_sampling_args(p: argparse.ArgumentParser, cfg_scale: float = 4.0, timestep_shift: float = 3.0) -> None:
    g = p.add_argument_group("sampling")
    g.add_argument("--cfg_scale", type=float, default=cfg_scale)
    g.add_argument("--cfg_norm", default="none", choices=CFG_NORMS)
    g.add_argument("--cfg_interval", type=float, nargs=2, default=[0.0, 1.0], metavar=("LO", "HI"),
                   help="guidance is applied for denoising times in [LO, HI]")
    g.add_argument("--timestep_shift", type=float, default=timestep_shift)
    g.add_argument("--num_steps", type=int, default=50)
    g.add_argument("--batch_size", type=int, default=1)
    g.add_argument("--seed", type=int, default=42)


def add_text_sampling_args(p: argparse.ArgumentParser) -> None:
    g = p.add_argument_group("text sampling")
    g.add_argument("--max_new_tokens", type=int, default=512)
    g.add_argument("--do_sample", action="store_true")
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--top_p", type=float, default=1.0)
    g.add_argument("--top_k", type=int, default=0)
    g.add_argument("--repetition_penalty", type=float, default=1.0)


def generation_config(a) -> Dict[str, Any]:
    return dict(max_new_tokens=a.max_new_tokens, do_sample=a.do_sample, temperature=a.temperature, top_p=a.top_p,
                top_k=a.top_k, repetition_penalty=a.repetition_penalty, seed=getattr(a, "seed", None))


# ---------------------------------------------------------------------------------------------------------------
# loading
# ---------------------------------------------------------------------------------------------------------------
def parse_max_memory(text: str) -> Dict:
    out: Dict = {}
    for part in (text or "").replace(";", ",").split(","):
        part = part.strip()
        if not part:
            continue
        if "=" not in part:
            raise ValueError(f"--max_memory entries look like 0=20GiB or cpu=64GiB, got {part!r}")
        k, v = (x.strip() for x in part.split("=", 1))
        out[int(k) if k.isdigit() else k] = v
    return out


def load_lora_state(path: str) -> Dict:
    p = Path(path)
    if p.is_dir():
        cands = sorted(p.glob("*.safetensors")) or sorted(p.glob("*.pt")) + sorted(p.glob("*.bin"))
        if not cands:
            raise FileNotFoundError(f"no LoRA weight file in {path}")
        p = cands[0]
    if p.suffix == ".safetensors":
        from safetensors.torch import load_file
        return load_file(str(p))
    import torch
    return torch.load(str(p), map_location="cpu")


def load_from_args(a):
    """(model, tokenizer) from the model / memory flags."""
    import torch
    import sensenova_u1_b200 as pkg
    from ..inference.api import ByteTokenizer, set_attn_backend
    from ..utils.offload import fast_mode_budget
    set_attn_backend(a.attn_backend if a.attn_backend != "sm100" else "auto")
    dt = getattr(torch, a.dtype)
    dev = a.device if a.device_map in ("none", "auto", "", None) else a.device_map
    okw = None
    if a.vram_mode == "fast":
        okw = {"resident_budget_bytes": fast_mode_budget(dev, a.fast_vram_fraction, a.fast_vram_headroom_gib,
                                                         a.fast_activation_reserve_gib, a.fast_vram_budget_gib)}
    if a.model_path:
        caps = parse_max_memory(a.max_memory)
        model = pkg.NEOChatModel.from_pretrained(a.model_path, device_map=dev, torch_dtype=dt, max_memory=caps or None,
                                                 vram_mode=None if (caps and a.vram_mode == "full") else a.vram_mode,
                                                 offload_kwargs=okw)
        try:
            from transformers import AutoTokenizer
            from ..inference.hf import resolve_checkpoint_path
            tok = AutoTokenizer.from_pretrained(resolve_checkpoint_path(a.model_path), trust_remote_code=False)
        except Exception:
            tok = ByteTokenizer(model.cfg.vocab_size)
    else:
        from ..config import get_config
        preset = a.random_init or "8b-mot"
        kw = {"num_layers": a.layers} if a.layers else {}
        if preset == "tiny-mot":           # the CUDA kernels want head size 128 and 16-pixel patches (32-pixel tokens)
            kw.setdefault("head_dim", 128)
            kw.setdefault("patch_size", 16)
        cfg = get_config(preset, **kw)
        model = pkg.NEOChatModel.from_config(cfg, device=dev, vram_mode=a.vram_mode, dtype=dt, offload_kwargs=okw)
        tok = ByteTokenizer(cfg.vocab_size)
    if a.gguf_checkpoint:
        from .gguf_loader import load_gguf
        load_gguf(a.gguf_checkpoint, model.store)
    if a.lora_path:
        from .lora import merge_lora
        n = merge_lora(model.store, load_lora_state(a.lora_path))
        print(f"merged {n} LoRA pairs from {a.lora_path}")
    return model, tok


# ---------------------------------------------------------------------------------------------------------------
# jobs and outputs
# ---------------------------------------------------------------------------------------------------------------
def read_jsonl(path: str) -> List[dict]:
    with open(path, encoding="utf-8") as f:
        return [json.loads(line) for line in f if line.strip()]


def iter_jobs(a, single: Dict[str, Any], required: Sequence[str] = ("prompt",)) -> Iterator[Tuple[Dict[str, Any], Path]]:
    """Yields (job, output path).  ``--jsonl``: one job per line (keys override the command-line values of the same
    name; outputs go to ``--output_dir`` as ``<index>.png`` or the line's ``output`` / ``id``); otherwise the single
    job described by the flags, written to ``--output``."""
    if getattr(a, "jsonl", None):
        out_dir = Path(a.output_dir)
        out_dir.mkdir(parents=True, exist_ok=True)
        for i, rec in enumerate(read_jsonl(a.jsonl)):
            for k in required:
                if k not in rec:
                    raise ValueError(f"{a.jsonl} line {i + 1}: missing {k!r}")
            job = dict(single)
            job.update(rec)
            name = str(rec.get("output") or rec.get("id") or f"{i:05d}")
            yield job, out_dir / (name if name.lower().endswith((".png", ".jpg", ".txt", ".json")) else name + ".png")
    else:
        yield dict(single), Path(a.output)


def warn_if_unsupported_resolution(width: int, height: int) -> Optional[str]:
    if (width, height) in SUPPORTED_RESOLUTIONS or width * height <= 1024 * 1024:
        return None
    msg = (f"{width}x{height} is not one of the resolution buckets the released checkpoints were trained on: "
           + ", ".join(f"{w}x{h}" for w, h in SUPPORTED_RESOLUTIONS))
    print("warning:", msg)
    return msg


def save_images(img, path: Path) -> List[Path]:
    """Writes a [B,3,H,W] batch in [-1,1]; several images get ``_i`` suffixes."""
    from ..inference.images import to_pil
    path.parent.mkdir(parents=True, exist_ok=True)
    out = []
    for i in range(img.shape[0]):
        p = path if img.shape[0] == 1 else path.with_name(f"{path.stem}_{i}{path.suffix}")
        to_pil(img[i]).save(p)
        out.append(p)
    return out


def build_enhancer(enabled: bool, style: str = "default"):
    """Prompt enhancer configured by U1_ENHANCE_{BACKEND,ENDPOINT,API_KEY,MODEL} (None when disabled)."""
    if not enabled:
        return None
    from ..inference.prompt_enhance import PromptEnhancer
    return PromptEnhancer.from_env(style=style)


def maybe_enhance(enhancer, prompt: str, verbose: bool = False, images=()) -> str:
    if enhancer is None:
        return prompt
    out = enhancer.enhance(prompt, images=images)
    if verbose:
        print("enhanced prompt:", out)
    return out


def is_main_rank() -> bool:
    return int(os.environ.get("RANK", "0")) == 0
