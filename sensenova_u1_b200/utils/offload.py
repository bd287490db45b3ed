"""Layer offload for inference on small devices: decoder-layer weights live in pinned host memory
and are streamed to the device ahead of use on a copy stream, with MoT-aware groups — during image
denoising only the generation-branch tensors of a layer are needed, during the prefix only the
understanding-branch ones (reference: src/sensenova_u1/utils/layer_offload.py:195-241, 465-998;
``--vram_mode`` presets and ``--max_memory`` caps: utils/offload.py:32-253,
utils/checkpoint_loading.py:236-245).

Three tiers of residency, all expressed in bytes so that a device budget maps onto them directly:

* resident layers: both branches stay on the device for the life of the model;
* generation residency: denoising runs the generation branch of every layer 50+ times per image, so
  on entering the ``denoise`` phase the generation tensors of as many streamed layers as the budget
  allows are copied once and kept until the phase changes;
* streaming slots: everything else passes through ``prefetch + 1`` slots, copied ``prefetch`` layers
  ahead on a side stream.

The stacked MoT layout makes a branch group one contiguous slice: ``tensor[0]`` (understanding) or
``tensor[1]`` (generation) of every per-layer parameter; the two expert mixtures of an MoE layer are
whole tensors of one branch each (``moe_und.*`` / ``moe_gen.*``).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch

from ..models.params import GEN, UND, ParamStore

# fraction of the layers that stay resident, fraction whose generation branch is kept during denoising, prefetch depth
VRAM_MODES = {"full": dict(resident_layers=None, gen_resident=0.0, prefetch=0),
              "fast": dict(resident_layers=0.5, gen_resident=0.5, prefetch=2),
              "balanced": dict(resident_layers=0.1, gen_resident=0.0, prefetch=1),
              "low": dict(resident_layers=0.0, gen_resident=0.0, prefetch=1)}


def parse_bytes(v) -> int:
    """``"20GiB"`` / ``"512MB"`` / ``1e9`` -> bytes (the spellings ``--max_memory`` accepts)."""
    if isinstance(v, (int, float)):
        return int(v)
    m = re.fullmatch(r"\s*([0-9.]+)\s*([KMGT]?)(i?)B?\s*", str(v), re.I)
    if not m:
        raise ValueError(f"cannot read a memory size from {v!r}")
    mult = {"": 0, "K": 1, "M": 2, "G": 3, "T": 4}[m.group(2).upper()]
    base = 1024 if m.group(3) else 1000
    return int(float(m.group(1)) * base ** mult)


def vram_mode_for_budget(max_memory: Dict, checkpoint_bytes: int, device: torch.device) -> str:
    """Preset for a ``max_memory`` cap of the target GPU: everything resident if the checkpoint plus working
    memory fits, otherwise the deepest residency that does (reference table: docs/gpu_mem_profiler.md:177-219)."""
    key = device.index if device.index is not None else 0
    cap = max_memory.get(key, max_memory.get(str(key), max_memory.get("cuda", None)))
    if cap is None:
        return "full"
    cap = parse_bytes(cap)
    work = 3 << 30                                    # caches, activations of a 2048 x 2048 image, workspaces
    if cap >= checkpoint_bytes + work:
        return "full"
    if cap >= 0.55 * checkpoint_bytes + work:
        return "fast"
    if cap >= 0.15 * checkpoint_bytes + work:
        return "balanced"
    return "low"


def fast_mode_budget(device, fraction: float = 0.9, headroom_gib: float = 2.0, activation_reserve_gib: float = 4.0,
                     explicit_budget_gib: float = 0.0, mem_info=None) -> int:
    """Bytes of decoder-layer weights the "fast" mode may keep on the device (the reference's automatic budget,
    src/sensenova_u1/utils/layer_offload.py:508-585): an explicit budget if given, otherwise ``fraction`` of the
    device's memory but not more than what is free now minus ``headroom``; the activation reserve (caches and
    working buffers of the largest request) comes off in both cases.  ``mem_info`` = (free, total) overrides the
    query (tests, CPU)."""
    import math
    if not (math.isfinite(fraction) and 0 < fraction <= 1):
        raise ValueError("fraction must satisfy 0 < value <= 1")
    for name, v in (("headroom_gib", headroom_gib), ("activation_reserve_gib", activation_reserve_gib),
                    ("explicit_budget_gib", explicit_budget_gib)):
        if not math.isfinite(v) or v < 0:
            raise ValueError(f"{name} must be finite and >= 0")
    gib = 1 << 30
    if mem_info is None:
        dev = torch.device(device)
        mem_info = torch.cuda.mem_get_info(dev) if dev.type == "cuda" and torch.cuda.is_available() else (0, 0)
    free, total = mem_info
    if explicit_budget_gib > 0:
        budget = int(explicit_budget_gib * gib)
    else:
        budget = min(int(total * fraction), max(0, int(free - headroom_gib * gib)))
    return max(0, budget - int(activation_reserve_gib * gib))


@dataclass
class _Slot:
    layer: int = -1
    branch: int = -1
    event: Optional[torch.cuda.Event] = None
    tensors: Optional[Dict[str, torch.Tensor]] = None


def _piece(name: str, t: torch.Tensor, br: int):
    """The part of per-layer tensor ``name`` that branch ``br`` uses (None: not used by that branch)."""
    if name.startswith("moe_und."):
        return t if br == UND else None
    if name.startswith("moe_gen."):
        return t if br == GEN else None
    return t[br] if t.dim() >= 2 and t.shape[0] == 2 else t


class LayerOffloader:
    """Serves the decoder-layer weights of one branch at a time from the three residency tiers.

    ``vram_mode`` picks a preset; ``resident_budget_bytes`` / ``gen_resident_budget_bytes`` override the
    preset's fractions with explicit device budgets.  ``on_phase`` callbacks are called with "prefix" /
    "denoise" whenever the phase changes (the reference's phase hook, layer_offload.py:465-520)."""

    def __init__(self, store: ParamStore, device, vram_mode: str = "balanced",
                 resident_budget_bytes: Optional[int] = None, gen_resident_budget_bytes: Optional[int] = None,
                 prefetch: Optional[int] = None):
        if vram_mode not in VRAM_MODES:
            raise ValueError(f"vram_mode must be one of {sorted(VRAM_MODES)}")
        self.cfg, self.device = store.cfg, torch.device(device)
        if self.cfg.is_moe and self.cfg.ep_size > 1:
            raise NotImplementedError("layer offload holds whole layers on one device; expert-parallel checkpoints run resident")
        mode = VRAM_MODES[vram_mode]
        L = self.cfg.num_layers
        self.names = [s.name.split(".", 2)[2] for s in store.specs if s.name.startswith("layers.0.")]
        per_layer = {n: store.p[f"layers.0.{n}"] for n in self.names}
        self.layer_bytes = sum(t.numel() * t.element_size() for t in per_layer.values())
        self.gen_layer_bytes = sum(p.numel() * p.element_size() for n, t in per_layer.items()
                                   if (p := _piece(n, t, GEN)) is not None)
        if resident_budget_bytes is not None:
            self.n_resident = min(L, int(resident_budget_bytes // max(1, self.layer_bytes)))
        else:
            frac = mode["resident_layers"]
            self.n_resident = L if frac is None else int(L * frac)
        streamed = L - self.n_resident
        if gen_resident_budget_bytes is not None:
            self.n_gen_resident = min(streamed, int(gen_resident_budget_bytes // max(1, self.gen_layer_bytes)))
        else:
            self.n_gen_resident = int(streamed * mode["gen_resident"])
        self.prefetch = mode["prefetch"] if prefetch is None else int(prefetch)
        cuda = self.device.type == "cuda"
        self.host: List[Dict[str, torch.Tensor]] = []
        self.resident: Dict[int, Dict[str, torch.Tensor]] = {}
        for l in range(L):
            d = {n: store.p[f"layers.{l}.{n}"] for n in self.names}
            if l < self.n_resident:
                self.resident[l] = {n: t.to(self.device) for n, t in d.items()}
                self.host.append({})
            else:
                self.host.append({n: (t.detach().cpu().pin_memory() if cuda else t.detach().cpu()) for n, t in d.items()})
        self.gen_cache: Dict[int, Dict[str, torch.Tensor]] = {}
        self.slots = [_Slot() for _ in range(self.prefetch + 1)]
        self.stream = torch.cuda.Stream(device=self.device) if cuda else None
        self.phase = "prefix"
        self.on_phase: List[Callable[[str], None]] = []
        self.bytes_streamed = 0

    # ---- phases ------------------------------------------------------------------------------------------
    def set_phase(self, phase: str):
        """'prefix' serves understanding-branch tensors, 'denoise' generation-branch ones."""
        if phase not in ("prefix", "denoise"):
            raise ValueError(phase)
        if phase == self.phase:
            return
        self.phase = phase
        if phase == "prefix":
            self.gen_cache.clear()                  # the generation residency is released with the phase
        for cb in self.on_phase:
            cb(phase)

    def _branch(self):
        return UND if self.phase == "prefix" else GEN

    def residency(self) -> Dict[str, int]:
        """Device bytes held by each tier right now."""
        held = lambda d: sum(t.numel() * t.element_size() for t in d.values())
        return {"resident": sum(held(d) for d in self.resident.values()),
                "generation": sum(held(d) for d in self.gen_cache.values()),
                "slots": sum(held(s.tensors) for s in self.slots if s.tensors)}

    # ---- copies --------------------------------------------------------------------------------------------
    def _copy_in(self, layer: int, br: int):
        out = {}
        for n, t in self.host[layer].items():
            piece = _piece(n, t, br)
            if piece is None:
                continue
            out[n] = piece.to(self.device, non_blocking=True)
            self.bytes_streamed += piece.numel() * piece.element_size()
        return out

    def _load(self, layer: int, slot: _Slot):
        br = self._branch()
        if self.stream is not None:
            # the slot being replaced may still be read by kernels already queued on the compute stream
            self.stream.wait_stream(torch.cuda.current_stream())
        ctx = torch.cuda.stream(self.stream) if self.stream is not None else _null()
        with ctx:
            out = self._copy_in(layer, br)
            if self.stream is not None:
                slot.event = torch.cuda.Event()
                slot.event.record(self.stream)
        slot.layer, slot.branch, slot.tensors = layer, br, out

    def layer_weights(self, layer: int) -> Dict[str, torch.Tensor]:
        """Branch tensors of ``layer`` on the device; starts the copy of the following layers."""
        br = self._branch()
        if layer in self.resident:
            return {n: p for n, t in self.resident[layer].items() if (p := _piece(n, t, br)) is not None}
        if br == GEN and layer in self.gen_cache:
            return self.gen_cache[layer]
        L = self.cfg.num_layers
        keep_gen = br == GEN and len(self.gen_cache) < self.n_gen_resident
        want = [l for l in range(layer, min(L, layer + self.prefetch + 1))
                if l not in self.resident and not (br == GEN and l in self.gen_cache)]
        for l in want:
            if not any(s.layer == l and s.branch == br for s in self.slots):
                victim = next((s for s in self.slots if s.layer not in want or s.branch != br), self.slots[0])
                self._load(l, victim)
        slot = next(s for s in self.slots if s.layer == layer and s.branch == br)
        if slot.event is not None:
            cur = torch.cuda.current_stream()
            cur.wait_event(slot.event)
            for t in slot.tensors.values():
                t.record_stream(cur)        # allocated on the copy stream, consumed on the compute stream
        tensors = slot.tensors
        if keep_gen:
            # promote to the generation residency: the slot forgets the tensors, the cache keeps them
            self.gen_cache[layer] = tensors
            slot.layer, slot.branch, slot.tensors, slot.event = -1, -1, None, None
        return tensors


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
