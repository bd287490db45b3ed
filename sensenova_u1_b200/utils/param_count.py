"""Parameter inventory by function: which weights serve understanding, which generation, which
both.  Groups follow the reference's report (src/sensenova_u1/utils/param_count.py:48-110,
docs/parameter_breakdown.md): visual understanding front-end, generation-only modules (generation
front-end, flow-matching head, timestep / noise-scale embedders), the generation and understanding
halves of the decoder, and the shared token embedding / LM head.

    python -m sensenova_u1_b200.utils.param_count --model 8b-mot [--json]
    python -m sensenova_u1_b200.utils.param_count --model_path CKPT [--custom_groups_json rules.json] [--show_groups shared]

With ``--model_path`` the tensors of a Hugging Face checkpoint directory are counted from the safetensors headers
(names, shapes, dtypes: no weight is read), grouped by name prefix as the reference's inspector does
(scripts/inspect_model_params.py, src/sensenova_u1/utils/param_count.py:57-140): generation transformer
(``fm_modules.*`` and every ``language_model.*`` tensor with ``_mot_gen``), shared (token embedding, LM head),
understanding transformer (the rest of ``vision_model.*`` / ``language_model.*``); ``--custom_groups_json`` replaces
the rules with ``{"group": ["prefix", ...]}``; ``--show_groups`` lists the members of the named groups, largest first.
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


# (group, prefixes, substrings that must occur): first match wins
DEFAULT_RULES = (("generation_transformer", ("fm_modules",), ()), ("generation_transformer", ("language_model",), ("_mot_gen",)),
                 ("shared", ("language_model.model.embed_tokens", "language_model.lm_head"), ()),
                 ("understanding_transformer", ("vision_model",), ()), ("understanding_transformer", ("language_model",), ()))
_DTYPE_BYTES = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1, "F8_E4M3": 1,
                "F8_E5M2": 1}


def load_rules(path=None):
    if not path:
        return DEFAULT_RULES
    with open(path, encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict) or not all(isinstance(v, list) and all(isinstance(x, str) for x in v) for v in raw.values()):
        raise ValueError('group rules are a JSON object {"group": ["prefix", ...]}')
    return tuple((g, tuple(v), ()) for g, v in raw.items())


def group_of(name: str, rules) -> str:
    for g, prefixes, contains in rules:
        if (not prefixes or name.startswith(prefixes)) and (not contains or any(c in name for c in contains)) \
                and (prefixes or contains):
            return g
    return "embedding_misc" if "embed" in name.lower() else "other"


def checkpoint_tensors(model_dir: str):
    """(name, shape, dtype tag) of every tensor in the ``*.safetensors`` files of a directory, from the file headers."""
    import struct
    from pathlib import Path
    files = sorted(Path(model_dir).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no *.safetensors in {model_dir}")
    seen = set()
    for f in files:
        with open(f, "rb") as fh:
            n = struct.unpack("<Q", fh.read(8))[0]
            header = json.loads(fh.read(n))
        for name, meta in header.items():
            if name == "__metadata__" or name in seen:
                continue
            seen.add(name)
            yield name, tuple(meta["shape"]), meta["dtype"]


def si(n: float, units=(("B", 1e9), ("M", 1e6), ("K", 1e3))) -> str:
    for suf, base in units:
        if abs(n) >= base:
            return f"{n / base:.3f}{suf}"
    return str(int(n))


def inspect_checkpoint(model_dir: str, rules=DEFAULT_RULES) -> dict:
    groups: Dict[str, dict] = {}
    total = total_bytes = 0
    for name, shape, dt in checkpoint_tensors(model_dir):
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = numel * _DTYPE_BYTES.get(dt, 2)
        g = groups.setdefault(group_of(name, rules), {"params": 0, "bytes": 0, "entries": []})
        g["params"] += numel
        g["bytes"] += nbytes
        g["entries"].append({"name": name, "numel": numel, "dtype": dt, "bytes": nbytes})
        total += numel
        total_bytes += nbytes
    for g in groups.values():
        g["entries"].sort(key=lambda e: -e["numel"])
    return {"model_path": model_dir, "total_params": total, "total_bytes": total_bytes,
            "groups": dict(sorted(groups.items(), key=lambda kv: -kv[1]["params"]))}


def checkpoint_report(res: dict, show=("shared",)) -> str:
    gb = (("GB", 1e9), ("MB", 1e6), ("KB", 1e3))
    lines = [f"{res['model_path']}: {si(res['total_params'])} parameters, {si(res['total_bytes'], gb)}"]
    for g, v in res["groups"].items():
        lines.append(f"  {g:28s} {si(v['params']):>10s}  {100.0 * v['params'] / max(1, res['total_params']):5.1f} %  {si(v['bytes'], gb):>10s}")
    for g in (res["groups"] if "all" in show else show):
        if g in res["groups"]:
            lines.append(f"\n[{g}]")
            lines += [f"  {e['numel']:>14,d}  {e['dtype']:5s} {e['name']}" for e in res["groups"][g]["entries"]]
    return "\n".join(lines)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="8b-mot")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--model_path", default=None, help="checkpoint directory (or hub id with a complete local snapshot) to count")
    ap.add_argument("--custom_groups_json", default=None)
    ap.add_argument("--show_groups", default="shared", help="comma-separated groups whose members are listed; all; empty: none")
    ap.add_argument("--dtype", default="bfloat16", help="accepted for compatibility: nothing is loaded, counts do not depend on it")
    a = ap.parse_args(argv)
    if a.model_path:
        from ..inference.hf import resolve_checkpoint_path
        res = inspect_checkpoint(resolve_checkpoint_path(a.model_path), load_rules(a.custom_groups_json))
        if a.json:
            print(json.dumps({k: (v if k != "groups" else {g: {x: y for x, y in gv.items() if x != "entries"} for g, gv in v.items()})
                              for k, v in res.items()}))
        else:
            print(checkpoint_report(res, tuple(x.strip() for x in a.show_groups.split(",") if x.strip())))
        return res
    cfg = get_config(a.model)
    if a.json:
        print(json.dumps({"model": cfg.name, "groups": breakdown(cfg), "active": active_params(cfg)}))
    else:
        print(report(cfg))


if __name__ == "__main__":
    main()
