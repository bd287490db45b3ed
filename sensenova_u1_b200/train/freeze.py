"""Freeze policy: which parameters train.

Reference semantics (training/sensenovavl/train/pipeline.py:176-224): ``freeze_backbone`` freezes the
understanding pixel front-end, ``freeze_llm`` freezes the whole language model (embedding, decoder
layers, final norm, LM head), ``unfreeze_lm_head`` re-enables the LM head and ``unfreeze_mot_gen``
re-enables every generation-branch ("mot_gen") tensor; the generation modules outside the language
model (generation front-end, timestep / noise embedders, flow-matching head) always train.

Here MoT tensors are stacked ``[understanding, generation]``, so a policy is a list of element ranges
per arena: the optimizer gives frozen ranges learning rate and weight decay 0, and the trainer clears
their gradients before the reduction so that they do not enter the clipping norm either.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

from ..models.params import GEN, ParamStore


def frozen_ranges(store: ParamStore, freeze_llm: bool = False, freeze_backbone: bool = False,
                  unfreeze_lm_head: bool = False, unfreeze_mot_gen: bool = False) -> Dict[str, List[Tuple[int, int]]]:
    """Element ranges [start, end) per arena that must not be updated (merged, sorted)."""
    out: Dict[str, List[Tuple[int, int]]] = {a: [] for a in store.sizes}

    def add(arena, s, e):
        if e > s:
            lst = out[arena]
            if lst and lst[-1][1] == s:
                lst[-1] = (lst[-1][0], e)
            else:
                lst.append((s, e))

    for spec in store.specs:
        arena, off = store.offsets[spec.name]
        n = spec.name
        end = off + spec.numel
        if n.startswith("vision_und."):
            if freeze_backbone:
                add(arena, off, end)
            continue
        in_llm = n in ("embed_tokens", "lm_head", "final_norm") or n.startswith("layers.") or n.startswith("mtp.")
        if not in_llm or not freeze_llm:
            continue
        if n == "lm_head" and unfreeze_lm_head:
            continue
        if ".moe_gen." in n:
            if not unfreeze_mot_gen:
                add(arena, off, end)
            continue
        dual = len(spec.shape) >= 2 and spec.shape[0] == 2 and n not in ("embed_tokens", "lm_head") and ".moe_" not in n
        if dual and unfreeze_mot_gen:
            half = spec.numel // 2
            lo = off + (1 - GEN) * half          # the understanding half stays frozen
            add(arena, lo, lo + half)
        else:
            add(arena, off, end)
    return out


def count_frozen(ranges: Dict[str, List[Tuple[int, int]]]) -> int:
    return sum(e - s for lst in ranges.values() for s, e in lst)
