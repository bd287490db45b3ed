"""LoRA merge into the base weights: W += (alpha / rank) * up @ down
(reference: src/sensenova_u1/utils/lora.py:14-49).  Adapter keys use the HF module names
(``...q_proj.lora_A.weight`` / ``lora_B.weight`` or ``lora_down`` / ``lora_up``); fused tensors
of this package (wqkv, w13) receive the update in the matching row range."""
from __future__ import annotations

import re
from typing import Dict

import torch

from ..models.params import ParamStore, hf_state_dict


def merge_lora(store: ParamStore, lora_sd: Dict[str, torch.Tensor], alpha: float = None, scale: float = 1.0) -> int:
    """Merges every adapter pair found in ``lora_sd``; returns the number of merged matrices."""
    views = hf_state_dict(store)          # HF name -> view into the arenas (fused tensors are sliced views)
    pairs: Dict[str, Dict[str, torch.Tensor]] = {}
    for k, v in lora_sd.items():
        m = re.match(r"(?:base_model\.model\.)?(.*)\.(lora_A|lora_B|lora_down|lora_up)(?:\.default)?\.weight$", k)
        if m:
            kind = "down" if m.group(2) in ("lora_A", "lora_down") else "up"
            pairs.setdefault(m.group(1), {})[kind] = v
        elif k.endswith(".alpha"):
            pairs.setdefault(k[:-6].replace("base_model.model.", ""), {})["alpha"] = v
    n = 0
    for mod, pr in pairs.items():
        if "down" not in pr or "up" not in pr:
            continue
        target = views.get(mod + ".weight")
        if target is None:
            raise KeyError(f"LoRA target {mod} not found in the model")
        rank = pr["down"].shape[0]
        a = float(pr["alpha"]) if "alpha" in pr else (alpha if alpha is not None else rank)
        delta = (pr["up"].float() @ pr["down"].float()) * (a / rank) * scale
        target.copy_((target.float() + delta.to(target.device).reshape(target.shape)).to(target.dtype))
        n += 1
    return n
