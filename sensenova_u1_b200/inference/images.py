"""Image pre/post-processing: native-resolution resize to a multiple of the token size within
a pixel budget, normalisation, tensor <-> PIL (reference: src/sensenova_u1/models/neo_unify/
utils.py:48-161, examples/t2i/inference.py:35-73)."""
from __future__ import annotations

import math
from typing import Tuple

import torch

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)

# (width, height) buckets of the text-to-image example, all multiples of 32 around 4 MPix
T2I_RESOLUTIONS = {"1:1": (2048, 2048), "16:9": (2720, 1536), "9:16": (1536, 2720), "3:2": (2496, 1664),
                   "2:3": (1664, 2496), "4:3": (2368, 1760), "3:4": (1760, 2368), "1:2": (1440, 2880),
                   "2:1": (2880, 1440), "1:3": (1152, 3456), "3:1": (3456, 1152)}


def smart_resize(height: int, width: int, factor: int = 32, min_pixels: int = 65536,
                 max_pixels: int = 4194304) -> Tuple[int, int]:
    """(h, w) divisible by ``factor`` with h*w inside [min_pixels, max_pixels], aspect kept."""
    if max(height, width) / max(1, min(height, width)) > 200:
        raise ValueError("aspect ratio above 200 is not supported")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def load_image_native(img, factor: int = 32, min_pixels: int = 65536, max_pixels: int = 4194304,
                      normalize: str = "imagenet") -> torch.Tensor:
    """PIL image or path -> float tensor [3,H,W]; ``normalize`` 'imagenet' (understanding input)
    or 'pm1' ([-1, 1], generation / editing source)."""
    from PIL import Image
    if not isinstance(img, Image.Image):
        img = Image.open(img)
    img = img.convert("RGB")
    h, w = smart_resize(img.height, img.width, factor, min_pixels, max_pixels)
    img = img.resize((w, h), Image.BICUBIC)
    x = torch.frombuffer(bytearray(img.tobytes()), dtype=torch.uint8).view(h, w, 3).permute(2, 0, 1).float() / 255.0
    if normalize == "imagenet":
        mean = torch.tensor(IMAGENET_MEAN).view(3, 1, 1)
        std = torch.tensor(IMAGENET_STD).view(3, 1, 1)
        return (x - mean) / std
    return x * 2 - 1


def to_pil(x: torch.Tensor):
    """[-1,1] tensor [3,H,W] -> PIL image (x * 0.5 + 0.5, clamped)."""
    from PIL import Image
    a = (x.detach().float().cpu() * 0.5 + 0.5).clamp(0, 1).mul(255).round().to(torch.uint8).permute(1, 2, 0).contiguous()
    return Image.frombytes("RGB", (a.shape[1], a.shape[0]), a.numpy().tobytes())
