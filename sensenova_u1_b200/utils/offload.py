"""Layer offload for inference on small devices: decoder-layer weights live in pinned host memory
and are streamed to the device one layer ahead on a copy stream, with MoT-aware groups — during
image denoising only the generation-branch tensors of a layer are needed, during the prefix only
the understanding-branch ones (reference: src/sensenova_u1/utils/layer_offload.py:195-241, 465-998;
``--vram_mode`` presets utils/offload.py:32-103).

The stacked MoT layout makes a group one contiguous slice: ``tensor[0]`` (understanding) or
``tensor[1]`` (generation) of every per-layer parameter.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..models.params import GEN, UND, ParamStore

VRAM_MODES = {"full": dict(resident_layers=None, prefetch=0),
              "fast": dict(resident_layers=0.5, prefetch=2),
              "balanced": dict(resident_layers=0.1, prefetch=1),
              "low": dict(resident_layers=0.0, prefetch=1)}


@dataclass
class _Slot:
    layer: int = -1
    branch: int = -1
    event: Optional[torch.cuda.Event] = None
    tensors: Optional[Dict[str, torch.Tensor]] = None


class LayerOffloader:
    """Keeps ``resident`` layers on the device and streams the rest through ``prefetch + 1`` slots."""

    def __init__(self, store: ParamStore, device, vram_mode: str = "balanced"):
        if vram_mode not in VRAM_MODES:
            raise ValueError(f"vram_mode must be one of {sorted(VRAM_MODES)}")
        self.cfg, self.device = store.cfg, torch.device(device)
        if self.cfg.is_moe:
            raise NotImplementedError("layer offload streams the dense MoT layers; MoE checkpoints run resident")
        mode = VRAM_MODES[vram_mode]
        L = self.cfg.num_layers
        frac = mode["resident_layers"]
        self.n_resident = L if frac is None else int(L * frac)
        self.prefetch = mode["prefetch"]
        self.names = [s.name.split(".", 2)[2] for s in store.specs if s.name.startswith("layers.0.")]
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
        self.slots = [_Slot() for _ in range(self.prefetch + 1)]
        self.stream = torch.cuda.Stream(device=self.device) if cuda else None
        self.phase = "prefix"
        self.bytes_streamed = 0

    def set_phase(self, phase: str):
        """'prefix' streams understanding-branch tensors, 'denoise' generation-branch ones."""
        if phase not in ("prefix", "denoise"):
            raise ValueError(phase)
        self.phase = phase

    def _branch(self):
        return UND if self.phase == "prefix" else GEN

    def _load(self, layer: int, slot: _Slot):
        br = self._branch()
        src = self.host[layer]
        out = {}
        if self.stream is not None:
            # the slot being replaced may still be read by kernels already queued on the compute stream
            self.stream.wait_stream(torch.cuda.current_stream())
        ctx = torch.cuda.stream(self.stream) if self.stream is not None else _null()
        with ctx:
            for n, t in src.items():
                piece = t[br] if t.shape[0] == 2 and t.dim() >= 2 else t
                out[n] = piece.to(self.device, non_blocking=True)
                self.bytes_streamed += piece.numel() * piece.element_size()
            if self.stream is not None:
                slot.event = torch.cuda.Event()
                slot.event.record(self.stream)
        slot.layer, slot.branch, slot.tensors = layer, br, out

    def layer_weights(self, layer: int) -> Dict[str, torch.Tensor]:
        """Branch tensors of ``layer`` on the device; starts the copy of the following layers."""
        br = self._branch()
        if layer in self.resident:
            d = self.resident[layer]
            return {n: (t[br] if t.shape[0] == 2 and t.dim() >= 2 else t) for n, t in d.items()}
        L = self.cfg.num_layers
        want = [l for l in range(layer, min(L, layer + self.prefetch + 1)) if l not in self.resident]
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
        return slot.tensors


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
