"""GGUF checkpoints: read (de-quantising block formats on the fly) into the parameter arenas.

The reference keeps GGUF weights quantised behind diffusers' ``GGUFLinear`` and de-quantises in
every forward (src/sensenova_u1/utils/gguf_loader.py:50-114).  Here the tcgen05 GEMMs consume bf16
operands, so a GGUF file is de-quantised once at load time, tensor by tensor (peak host memory =
one tensor), into the bf16 arenas; tensor names are the HF names of the safetensors checkpoints.
"""
from __future__ import annotations

from typing import Dict, Iterator, List, Tuple

import torch


def iter_gguf_tensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yields (name, float32 tensor) for every tensor of a GGUF file."""
    import numpy as np
    import gguf
    from gguf import quants
    reader = gguf.GGUFReader(path)
    for t in reader.tensors:
        shape = [int(x) for x in reversed(t.shape.tolist())]      # GGUF stores dimensions innermost first
        if t.tensor_type in (gguf.GGMLQuantizationType.F32, gguf.GGMLQuantizationType.F16):
            arr = np.asarray(t.data).astype(np.float32)
        elif t.tensor_type == gguf.GGMLQuantizationType.BF16:
            raw = np.asarray(t.data).view(np.uint16).astype(np.uint32) << 16
            arr = raw.view(np.float32)
        else:
            arr = quants.dequantize(np.asarray(t.data), t.tensor_type)
        yield t.name, torch.from_numpy(np.ascontiguousarray(arr)).reshape(shape)


def load_gguf(path: str, store, strict: bool = False) -> List[str]:
    """Copies the tensors of a GGUF file into ``store`` (a ``ParamStore``); returns the HF names the
    file did not provide."""
    from ..models.params import hf_state_dict
    views = hf_state_dict(store)
    seen = set()
    for name, w in iter_gguf_tensors(path):
        v = views.get(name)
        if v is None:
            continue
        if v.numel() != w.numel():
            raise ValueError(f"{name}: GGUF tensor has {w.numel()} elements, model expects {v.numel()}")
        v.copy_(w.reshape(v.shape).to(v.dtype))
        seen.add(name)
    missing = [n for n in views if n not in seen]
    if strict and missing:
        raise KeyError(f"{len(missing)} tensors missing from {path}, e.g. {missing[:4]}")
    return missing


def save_gguf(path: str, state: Dict[str, torch.Tensor], quant: str = "F16", arch: str = "neo_unify") -> None:
    """Writes tensors to a GGUF file (``quant``: F32, F16 or Q8_0; 1-D tensors stay F32)."""
    import numpy as np
    import gguf
    from gguf import quants
    qt = getattr(gguf.GGMLQuantizationType, quant)
    w = gguf.GGUFWriter(path, arch)
    for name, t in state.items():
        a = t.detach().float().cpu().numpy()
        if a.ndim < 2 or quant == "F32" or (quant == "Q8_0" and a.shape[-1] % 32):
            w.add_tensor(name, a.astype(np.float32))
        elif quant == "F16":
            w.add_tensor(name, a.astype(np.float16))
        else:
            w.add_tensor(name, quants.quantize(a, qt), raw_shape=None, raw_dtype=qt)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
