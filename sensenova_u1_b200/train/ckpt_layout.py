"""Training-checkpoint tensor layout: name-keyed shards in the reference's training key names.

The reference's training checkpoints (training/sensenovalm/checkpoint/components.py:512-621) hold a
``state_dict`` keyed by module path, one file per weight-parallel rank, every linear weight split by
rows over the weight-parallel group (the token embedding by columns), norms and the small
flow-matching / vision front-end modules replicated.  Expert weights go to one file per
(MoE module, expert-parallel rank): ``model_moe_layer{2*l + gen}_expert{ep}_wp{w}.pt`` with the local
experts stacked along dim 0 in ``[in, out]`` orientation (components.py:134-181).  The reference's
``tools/revert2hf.py`` (:211-661) merges exactly this layout back into the HF checkpoint.

This module converts between that layout and the flat arenas of :class:`ParamStore`:

    train_state_dict(store)                -> {training key: full tensor}      (non-expert tensors)
    shard_state_dict(sd, wp_rank, wp_size) -> the rows / columns of one weight-parallel rank
    merge_shards([sd_0 .. sd_{wp-1}])      -> full tensors again
    load_train_state_dict(store, sd)       -> copies into the arenas
    expert_files(store) / load_expert_file(...)   per-rank expert tensors

Only tensor *names* and slicing rules are shared with the reference; the mapping is derived from
this package's own HF name table (``models/params.py::hf_state_dict``).
"""
from __future__ import annotations

import re
from typing import Dict, Iterable, List, Sequence, Tuple

import torch

from ..models.params import GEN, UND, ParamStore, hf_state_dict

PREFIX = "model."

# HF module path fragment -> training module path fragment (applied to non-expert tensors of a decoder layer)
_LAYER_RULES: Sequence[Tuple[str, str]] = (
    ("self_attn.q_proj", "attention.wq"), ("self_attn.k_proj", "attention.wk"), ("self_attn.v_proj", "attention.wv"),
    ("self_attn.o_proj", "attention.wo"), ("self_attn.q_norm", "attention.q_norm"), ("self_attn.k_norm", "attention.k_norm"),
    ("post_attention_layernorm", "ffn_norm"), ("input_layernorm", "attention_norm"),
)
_FFN_RULES: Sequence[Tuple[str, str]] = (("gate_proj", "w1"), ("up_proj", "w3"), ("down_proj", "w2"))


def hf_to_train_key(k: str) -> str:
    """``language_model.model.layers.3.mlp_mot_gen.up_proj.weight`` ->
    ``model.language_model.layers.3.feed_forward_mot_gen.w3.weight`` and so on."""
    if k == "language_model.model.embed_tokens.weight":
        return PREFIX + "language_model.tok_embeddings.weight"
    if k == "language_model.lm_head.weight":
        return PREFIX + "language_model.output.weight"
    m = re.fullmatch(r"language_model\.model\.(norm(?:_mot_gen)?\.weight)", k)
    if m:
        return PREFIX + "language_model." + m.group(1)
    m = re.fullmatch(r"language_model\.model\.layers\.(\d+)\.(.+)", k)
    if m:
        rest = m.group(2)
        mm = re.fullmatch(r"mlp(_mot_gen)?\.gate\.weight", rest)
        if mm:
            rest = f"feed_forward{mm.group(1) or ''}.moe_layer.gate.wg.weight"
        elif rest.startswith("mlp"):
            mm = re.fullmatch(r"mlp(_mot_gen)?\.(gate_proj|up_proj|down_proj)\.weight", rest)
            if mm is None:
                raise KeyError(f"no training name for {k}")
            rest = f"feed_forward{mm.group(1) or ''}.{dict(_FFN_RULES)[mm.group(2)]}.weight"
        else:
            for a, b in _LAYER_RULES:
                if rest.startswith(a):
                    rest = b + rest[len(a):]
                    break
        return PREFIX + f"language_model.layers.{m.group(1)}." + rest
    return PREFIX + k          # vision_model.*, fm_modules.*


def split_dim(train_key: str):
    """0 / 1: the dimension a weight-parallel group splits; None: replicated on every rank."""
    k = train_key
    if "tok_embeddings" in k:
        return 1
    if ("fm_modules" in k or "vision_model" in k or ".mtp_extra." in k or "language_model.norm" in k or "moe_layer.gate" in k
            or "_norm" in k):
        return None
    return 0


def train_state_dict(store: ParamStore) -> Dict[str, torch.Tensor]:
    """Every non-expert tensor under its training name (views into the arenas, full size)."""
    out = {}
    for k, v in hf_state_dict(store).items():
        if ".experts." in k:
            continue
        out[hf_to_train_key(k)] = v
    for name, t in store.p.items():
        if name.startswith("mtp."):       # multi-token-prediction heads: not part of the HF inference checkpoint
            out[PREFIX + "mtp_extra." + name] = t
    return out


def shard_state_dict(sd: Dict[str, torch.Tensor], wp_rank: int, wp_size: int) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        d = split_dim(k)
        if d is None or wp_size == 1:
            out[k] = v.detach().clone()
            continue
        n = v.shape[d]
        if n % wp_size:
            raise ValueError(f"{k}: dim {d} of size {n} does not split over {wp_size} weight-parallel ranks")
        out[k] = v.narrow(d, wp_rank * (n // wp_size), n // wp_size).detach().clone()
    return out


def merge_shards(shards: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    out = {}
    for k in shards[0]:
        d = split_dim(k)
        out[k] = shards[0][k] if (d is None or len(shards) == 1) else torch.cat([s[k] for s in shards], dim=d)
    return out


def load_train_state_dict(store: ParamStore, sd: Dict[str, torch.Tensor], strict: bool = True) -> List[str]:
    """Copies full (merged) training-named tensors into the arenas; returns the names not found."""
    missing = []
    for k, view in train_state_dict(store).items():
        src = sd.get(k, sd.get(k[len(PREFIX):]))
        if src is None:
            missing.append(k)
            continue
        view.copy_(src.to(view.dtype).reshape(view.shape) if view.is_contiguous() else src.to(view.dtype))
    if strict and missing:
        raise KeyError(f"{len(missing)} tensors missing from the training checkpoint, e.g. {missing[:4]}")
    return missing


# ---------------------------------------------------------------------------
# experts: one file per (layer, branch, expert-parallel rank)
# ---------------------------------------------------------------------------
def _expert_key(layer: int, gen: bool, which: str) -> str:
    ff = "feed_forward_mot_gen" if gen else "feed_forward"
    return PREFIX + f"language_model.layers.{layer}.{ff}.moe_layer.experts.wrapped_experts.0.{which}.weight"


def expert_file_name(layer: int, gen: bool, ep_rank: int, ewp_rank: int = 0) -> str:
    return f"model_moe_layer{2 * layer + (1 if gen else 0)}_expert{ep_rank}_wp{ewp_rank}.pt"


def expert_files(store: ParamStore) -> Iterable[Tuple[str, Dict[str, torch.Tensor]]]:
    """(file name, state dict) of this rank's experts: w1 / w3 ``[E_local * H, F]``, w2 ``[E_local * F, H]``
    (the ``[in, out]`` orientation of the reference's grouped expert weights)."""
    cfg = store.cfg
    if not cfg.is_moe:
        return
    Fe = cfg.moe_intermediate_size
    ep_rank = store.ep_rank if cfg.ep_size > 1 else 0
    for l in range(cfg.num_layers):
        for gen, br in ((False, "und"), (True, "gen")):
            w13, w2 = store.p[f"layers.{l}.moe_{br}.w13"], store.p[f"layers.{l}.moe_{br}.w2"]
            E = w13.shape[0]
            sd = {_expert_key(l, gen, "w1"): w13[:, :Fe].transpose(1, 2).reshape(E * cfg.hidden_size, Fe).detach().clone(),
                  _expert_key(l, gen, "w3"): w13[:, Fe:].transpose(1, 2).reshape(E * cfg.hidden_size, Fe).detach().clone(),
                  _expert_key(l, gen, "w2"): w2.transpose(1, 2).reshape(E * Fe, cfg.hidden_size).detach().clone()}
            yield expert_file_name(l, gen, ep_rank), sd


def load_expert_file(store: ParamStore, layer: int, gen: bool, sd: Dict[str, torch.Tensor]) -> None:
    cfg = store.cfg
    Fe, H = cfg.moe_intermediate_size, cfg.hidden_size
    br = "gen" if gen else "und"
    w13, w2 = store.p[f"layers.{layer}.moe_{br}.w13"], store.p[f"layers.{layer}.moe_{br}.w2"]
    E = w13.shape[0]

    def get(which):
        k = _expert_key(layer, gen, which)
        return sd[k] if k in sd else sd[k[len(PREFIX):]]
    w13[:, :Fe].copy_(get("w1").view(E, H, Fe).transpose(1, 2).to(w13.dtype))
    w13[:, Fe:].copy_(get("w3").view(E, H, Fe).transpose(1, 2).to(w13.dtype))
    w2.copy_(get("w2").view(E, Fe, H).transpose(1, 2).to(w2.dtype))


def model_config_record(cfg) -> dict:
    """``model_config.pt``: the fields the reference's converter reads (tools/revert2hf.py:497-506) next to this
    package's own configuration."""
    rec = {"num_layers": cfg.num_layers, "vit_cfg": {"num_hidden_layers": 0}, "hidden_size": cfg.hidden_size,
           "num_attention_heads": cfg.num_heads, "num_kv_attention_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
           "vocab_size": cfg.vocab_size, "model_config": dict(cfg.__dict__)}
    if cfg.is_moe:
        rec["moe_kwargs"] = {"num_experts": cfg.num_experts, "gen_num_experts": cfg.gen_num_experts,
                             "top_k": cfg.num_experts_per_tok, "first_k_dense_replace": 0,
                             "moe_intermediate_size": cfg.moe_intermediate_size}
    return rec
