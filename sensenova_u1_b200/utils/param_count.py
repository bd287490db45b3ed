"""Parameter inventory by function: which weights serve understanding, which generation, which
both.  Groups follow the reference's report (src/sensenova_u1/utils/param_count.py:48-110,
docs/parameter_breakdown.md): visual understanding front-end, generation-only modules (generation
front-end, flow-matching head, timestep / noise-scale embedders), the generation and understanding
halves of the decoder, and the shared token embedding / LM head.

    python -m sensenova_u1_b200.utils.param_count --model 8b-mot [--json]
"""
from __future__ import annotations

import argparse
import json
from collections import OrderedDict
from typing import Dict

from ..config import ModelConfig, get_config
from ..models.params import build_specs

GROUPS = ("visual_understanding", "generation_modules", "llm_generation", "llm_understanding", "shared")


def breakdown(cfg: ModelConfig) -> "OrderedDict[str, int]":
    """Parameter count per group (whole model: every expert of every rank)."""
    out = OrderedDict((g, 0) for g in GROUPS)
    ep = max(1, cfg.ep_size)
    for s in build_specs(cfg):
        n = s.numel * (ep if s.arena == "exp" else 1)
        name = s.name
        if name.startswith("vision_und."):
            out["visual_understanding"] += n
        elif name.startswith(("vision_gen.", "fm_head.", "timestep_embedder.", "noise_scale_embedder.")):
            out["generation_modules"] += n
        elif name in ("embed_tokens", "lm_head"):
            out["shared"] += n
        elif ".moe_gen." in name:
            out["llm_generation"] += n
        elif ".moe_und." in name:
            out["llm_understanding"] += n
        elif s.shape[0] == 2 and (name.startswith("layers.") or name.startswith("mtp.") or name == "final_norm"):
            # dual tensors: index 0 = understanding weights, 1 = generation weights
            out["llm_understanding"] += n // 2
            out["llm_generation"] += n - n // 2
        else:
            out["shared"] += n
    return out


def active_params(cfg: ModelConfig) -> Dict[str, int]:
    """Parameters a token actually passes through (one MoT branch; top-k experts for MoE)."""
    b = breakdown(cfg)
    und, gen = b["llm_understanding"], b["llm_generation"]
    if cfg.is_moe:
        Fe, H, L = cfg.moe_intermediate_size, cfg.hidden_size, cfg.num_layers
        per_expert = 3 * Fe * H
        und -= L * (cfg.num_experts - cfg.num_experts_per_tok) * per_expert
        gen -= L * (cfg.gen_num_experts - cfg.gen_num_experts_per_tok) * per_expert
    return {"understanding_token": und + b["shared"], "generation_token": gen + b["generation_modules"]}


def report(cfg: ModelConfig) -> str:
    b = breakdown(cfg)
    tot = sum(b.values())
    lines = [f"{cfg.name}: {tot / 1e9:.3f} B parameters"]
    for k, v in b.items():
        lines.append(f"  {k:24s} {v / 1e9:9.3f} B  {100.0 * v / tot:5.1f} %")
    for k, v in active_params(cfg).items():
        lines.append(f"  active per {k:19s} {v / 1e9:9.3f} B")
    return "\n".join(lines)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="8b-mot")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    cfg = get_config(a.model)
    if a.json:
        print(json.dumps({"model": cfg.name, "groups": breakdown(cfg), "active": active_params(cfg)}))
    else:
        print(report(cfg))


if __name__ == "__main__":
    main()
