"""Image conversions between ComfyUI's IMAGE type and this framework.

ComfyUI passes images as float tensors ``[B, H, W, 3]`` in [0, 1]; the model API takes and returns
``[3, H, W]`` / ``[B, 3, H, W]`` tensors in [-1, 1] (generation) and PNG / JPEG bytes travel over
HTTP.  (Role of the reference's apps/comfyui/image_utils.py:1-125.)
"""
from __future__ import annotations

import base64
import io
from typing import List

import torch

MAX_IMAGE_BYTES = 20 * 1024 * 1024


def comfy_to_model(image: torch.Tensor) -> List[torch.Tensor]:
    """``[B,H,W,3]`` in [0,1] -> list of ``[3,H,W]`` in [-1,1]."""
    if image.dim() == 3:
        image = image[None]
    if image.dim() != 4 or image.shape[-1] not in (3, 4):
        raise ValueError(f"expected a ComfyUI IMAGE [B,H,W,3], got {tuple(image.shape)}")
    x = image[..., :3].float().clamp(0, 1) * 2 - 1
    return [x[i].permute(2, 0, 1).contiguous() for i in range(x.shape[0])]


def model_to_comfy(images: torch.Tensor) -> torch.Tensor:
    """``[3,H,W]`` or ``[B,3,H,W]`` in [-1,1] -> ``[B,H,W,3]`` in [0,1] on the CPU."""
    if images.dim() == 3:
        images = images[None]
    return ((images.detach().float().cpu().clamp(-1, 1) + 1) * 0.5).permute(0, 2, 3, 1).contiguous()


def stack_for_comfy(images: List[torch.Tensor]) -> torch.Tensor:
    """Pictures of possibly different sizes -> one IMAGE batch (smaller ones are zero-padded to the
    largest, which is how a preview node can show an interleaved answer in one widget)."""
    if not images:
        return torch.zeros(1, 64, 64, 3)
    imgs = [model_to_comfy(i)[0] for i in images]
    H, W = max(i.shape[0] for i in imgs), max(i.shape[1] for i in imgs)
    out = torch.zeros(len(imgs), H, W, 3)
    for k, im in enumerate(imgs):
        out[k, : im.shape[0], : im.shape[1]] = im
    return out


def comfy_to_png_bytes(image: torch.Tensor, index: int = 0) -> bytes:
    from PIL import Image
    if image.dim() == 3:
        image = image[None]
    arr = (image[index, ..., :3].float().clamp(0, 1) * 255).round().to(torch.uint8).cpu().numpy()
    buf = io.BytesIO()
    Image.fromarray(arr, "RGB").save(buf, format="PNG")
    data = buf.getvalue()
    if len(data) > MAX_IMAGE_BYTES:
        raise ValueError(f"encoded image is {len(data)} bytes, above the {MAX_IMAGE_BYTES}-byte request limit")
    return data


def bytes_to_comfy(data: bytes) -> torch.Tensor:
    from PIL import Image
    import numpy as np
    im = Image.open(io.BytesIO(data)).convert("RGB")
    return torch.from_numpy(np.asarray(im).copy()).float().div(255.0)[None]


def data_url(image: torch.Tensor, index: int = 0) -> str:
    return "data:image/png;base64," + base64.b64encode(comfy_to_png_bytes(image, index)).decode()


def is_http_url(s: str) -> bool:
    return s.startswith("http://") or s.startswith("https://")


def describe(image: torch.Tensor) -> str:
    b, h, w, c = image.shape
    return f"batch={b} size={w}x{h} channels={c} min={float(image.min()):.3f} max={float(image.max()):.3f}"
